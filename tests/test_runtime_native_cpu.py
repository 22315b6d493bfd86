"""The native executor pieces: compute-graph hazards / levels / hash / alias groups, the fusion planner and the GEMM plan cache."""
import pytest

from oa_b200.runtime.graph import (OaAccess, OaComputeGraph, OaDnnEngineType, OaDnnGraph, OaDnnOpType, OaDnnPlanner, OaGemmPlanCache)

R, W, RW = OaAccess.Read, OaAccess.Write, OaAccess.ReadWrite


def _chain():
    g = OaComputeGraph()
    g.AddNode("a", [(1, 100, R), (2, 400, W)])           # 0: x -> t1
    g.AddNode("b", [(1, 100, R), (3, 400, W)])           # 1: x -> t2   (independent of 0)
    g.AddNode("c", [(2, 400, R), (3, 400, R), (4, 400, W)])   # 2: t1, t2 -> t3
    g.AddNode("d", [(4, 400, R), (5, 400, W)])           # 3: t3 -> t4  (t1, t2 dead: t4 can reuse their space)
    g.AddNode("e", [(2, 400, W)])                        # 4: overwrites t1: WAR on node 2
    return g


def test_hazards_levels_and_aliasing():
    g = _chain()
    assert g.NumNodes() == 5
    assert g.NodeDeps(0) == [] and g.NodeDeps(1) == []
    assert g.NodeDeps(2) == [0, 1] and g.NodeDeps(3) == [2]
    assert g.NodeDeps(4) == [0, 2]                       # WAW on its own earlier writer, WAR on the reader
    assert [g.NodeLevel(i) for i in range(5)] == [0, 0, 1, 2, 2]
    assert g.NumLevels() == 3 and g.NumBarriers() == 3
    naive, aliased = g.Memory()
    assert naive == 100 + 4 * 400 and aliased < naive
    groups = {b[0]: b[4] for b in g.Buffers()}
    assert groups[5] == groups[3]                        # t4 reuses t2's group (t2 died at node 2, t4 is born at node 3)
    assert groups[2] != groups[3]


def test_structural_hash_detects_any_change():
    a, b = _chain(), _chain()
    assert a.Hash() == b.Hash()
    b.AddNode("f", [(5, 400, R)])
    assert a.Hash() != b.Hash()
    c = OaComputeGraph()
    c.AddNode("a", [(1, 100, R), (2, 400, W)], push=b"\x01")
    d = OaComputeGraph()
    d.AddNode("a", [(1, 100, R), (2, 400, W)], push=b"\x02")
    assert c.Hash() != d.Hash() and c.Report()["nodes"] == 1


def _ffn_block():
    g = OaDnnGraph()
    for i, ext in ((0, True), (1, True), (2, True), (3, True)):
        assert g.AddMatrix(i, [64, 64], external=ext)
    for i in range(4, 20):
        assert g.AddMatrix(i, [64, 64])
    T = OaDnnOpType
    assert g.AddOp(T.Add, [0, 1], [4])                   # 0 residual add
    assert g.AddOp(T.RmsNorm, [4, 2], [5])               # 1 norm
    assert g.AddOp(T.Matmul, [5, 3], [6])                # 2 gate
    assert g.AddOp(T.Relu, [1], [12])                    # 3 unrelated op between the members of the pattern
    assert g.AddOp(T.Matmul, [5, 3], [7])                # 4 up
    assert g.AddOp(T.Silu, [6], [8])                     # 5
    assert g.AddOp(T.Multiply, [8, 7], [9])              # 6
    assert g.AddOp(T.Matmul, [9, 3], [10])               # 7 down
    assert g.AddOp(T.BiasAdd, [10, 2], [11])             # 8
    assert g.AddOp(T.Gelu, [11], [13])                   # 9
    assert g.AddOp(T.FlashAttentionCausal, [13], [14, 15])   # 10
    return g


def test_planner_finds_patterns_across_unrelated_ops():
    plan, st = OaDnnPlanner.Plan(_ffn_block(), allow_recompute=False)
    assert st and plan.PlannerAbi == 1
    by_engine = {p.Engine: p for p in plan.Partitions}
    E = OaDnnEngineType
    assert by_engine[E.ResidualNorm].Ops == [0, 1]
    assert by_engine[E.GatedFfn].Ops == [2, 4, 5, 6] and by_engine[E.GatedFfn].SavedForBackward == [5]
    assert by_engine[E.BlasLtEpilogue].Ops == [7, 8, 9] and by_engine[E.BlasLtEpilogue].SavedForBackward == [11]
    assert by_engine[E.FlashAttention].SavedForBackward == [14, 15]
    assert by_engine[E.Portable].Ops == [3]
    assert sorted(o for p in plan.Partitions for o in p.Ops) == list(range(11))
    again, _ = OaDnnPlanner.Plan(_ffn_block(), allow_recompute=False)
    assert again.GraphHash == plan.GraphHash


def test_planner_qkv_tensor_parallel_and_validation():
    T, E = OaDnnOpType, OaDnnEngineType
    g = OaDnnGraph()
    g.AddMatrix(0, [128, 64], external=True)
    g.AddMatrix(1, [64, 64], external=True)
    for i in (2, 3, 4):
        g.AddMatrix(i, [128, 64])
        g.AddOp(T.Matmul, [0, 1], [i])
    plan, st = OaDnnPlanner.Plan(g)
    assert st and [p.Engine for p in plan.Partitions] == [E.PackedQkv] and plan.Partitions[0].Ops == [0, 1, 2]
    g = OaDnnGraph()
    g.AddMatrix(0, [128, 64], external=True, row_sharded=True)
    g.AddMatrix(1, [64, 64], external=True)
    g.AddMatrix(2, [1024, 64])
    g.AddMatrix(3, [128, 64], row_sharded=True)
    g.AddOp(T.Matmul, [0, 1], [2])
    g.AddOp(T.Matmul, [2, 1], [3])
    plan, st = OaDnnPlanner.Plan(g)
    assert [p.Engine for p in plan.Partitions] == [E.AllGatherGemm, E.GemmReduceScatter]
    bad = OaDnnGraph()
    bad.AddMatrix(0, [4, 4])                             # not external and never produced
    bad.AddMatrix(1, [4, 4])
    bad.AddOp(T.Relu, [0], [1])
    plan, st = OaDnnPlanner.Plan(bad)
    assert plan is None and not st and "producer" in st.message
    assert not OaDnnGraph().AddMatrix(5, [0, 4])


def test_plan_cache_elects_by_median_and_persists(tmp_path):
    c = OaGemmPlanCache()
    assert c.Lookup(4096, 4096, 1024) is None
    for us in (100, 101, 300):                            # one outlier must not decide
        c.Record(4096, 4096, 1024, 256, 1, us)
    for us in (110, 111, 112):
        c.Record(4096, 4096, 1024, 128, 1, us)
    assert c.Lookup(4096, 4096, 1024) == (256, 1)
    med, p95, n = c.Timing(4096, 4096, 1024)
    assert med == pytest.approx(101) and n == 3
    c.Set(32, 4096, 4096, 128, 8, role=2, world=8)
    path = str(tmp_path / "gemm_route_cache.bin")
    assert c.Save(path)
    d = OaGemmPlanCache()
    assert d.Load(path) and d.Size() == 2 and d.Lookup(32, 4096, 4096, role=2, world=8) == (128, 8)
    raw = bytearray(open(path, "rb").read())
    raw[-3] ^= 1
    open(path, "wb").write(bytes(raw))
    e = OaGemmPlanCache()
    st = e.Load(path)
    assert not st and st.code.name == "DataLoss" and e.Size() == 0
    assert not e.Load(str(tmp_path / "missing.bin"))
    assert c.Stats()[0] >= 1


def test_kernel_registry_and_operation_contracts():
    from oa_b200.core import registry as R
    assert R.Fnv1a("") == 0xCBF29CE484222325 and R.Fnv1a("a") == 0xAF63DC4C8601EC8C          # FNV-1a 64 test vectors
    ks = R.OaKernelRegistry.All()
    assert len(ks) > 100 and len({k.Id for k in ks}) == len(ks) and len({k.Name for k in ks}) == len(ks)
    g = R.OaKernelRegistry.Find("oa_gemm_bf16_batched")
    assert g is not None and g.Provider == "gemm_tcgen05.cu" and R.OaKernelRegistry.FindById(g.Id).Name == g.Name
    same_cat = [k for k in ks if k.Category == g.Category]
    assert all(k.Id >> 16 == g.Id >> 16 for k in same_cat) and sorted(k.Id & 0xFFFF for k in same_cat) == list(range(len(same_cat)))
    assert R.OaKernelRegistry.Find("oa_rl_gae").Provider == "rl.cu" and R.OaKernelRegistry.Find("nope") is None
    ops = R.OaOperationRegistry.All()
    assert len(ops) > 80
    lin = R.OaOperationRegistry.Find("Linear")
    assert lin.Kind == R.OaOperationKind.Gemm and lin.Differentiation == R.OaDifferentiation.Analytic and lin.Lowering == R.OaLowering.Gemm
    assert lin.Hash == R.Fnv1a("Linear") and R.OaOperationRegistry.FindByHash(lin.Hash).Name == "Linear"
    assert R.OaOperationRegistry.Find("Zeros").Differentiation == R.OaDifferentiation.NoGradient
    assert R.OaOperationRegistry.Find("AddInPlace").Effects == R.OaEffects.MutatesInput
    assert R.OaOperationRegistry.Find("Dropout").Effects == R.OaEffects.Random
    assert R.OaOperationRegistry.Find("Loss.CrossEntropy").Kind == R.OaOperationKind.Loss
    assert R.OaOperationRegistry.Find("Tanh").Differentiation == R.OaDifferentiation.Analytic


def test_gemm_tuner_times_unknown_shapes_once_and_persists(tmp_path):
    """The launch-plan cache has a consumer: the tuner times each candidate tile of an unknown shape once, keeps the fastest,
    answers from the cache afterwards, and reloads its plans from a file (Runtime/GemmPlanCache.cpp)."""
    from oa_b200.runtime.gemm_tuner import OaGemmTuner
    cost = {0: 50.0, 128: 70.0, 256: 40.0}
    launched = []

    def timer(run, reps):
        run()
        return cost[launched[-1]]

    path = str(tmp_path / "plans.bin")
    t = OaGemmTuner(path, tune=True, reps=3, timer=timer)
    assert t.Plan(4096, 1024, 512, 0, 0, launched.append) == 256
    assert launched == [0, 128, 256] and t.Tuned == 1
    assert t.Plan(4096, 1024, 512, 0, 0, launched.append) == 256 and len(launched) == 3       # answered from the cache
    assert t.Plan(4096, 128, 512, 0, 0, launched.append) == 0                                  # 256 does not fit N = 128
    assert launched[3:] == [0, 128]
    med, p95, n = t.Cache.Timing(4096, 1024, 512)
    assert n >= 1 and med > 0
    t.Save()
    again = OaGemmTuner(path, tune=False)
    assert again.Plan(4096, 1024, 512, 0, 0, launched.append) == 256
    assert again.Plan(64, 64, 64, 0, 0, launched.append) == 0 and len(launched) == 5           # tuning off: library's choice
