"""Workspace arena, lifetime helpers, launch planner and the shape-only backend
(reference: `src/workspace.ts`, `src/heap.ts`, `src/using-holder.ts`, `src/tensor-tree.ts`,
`src/sparse-mla-planner.ts`, `src/meta_ops.ts`)."""
import pytest
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel, KVCacheTensors, make_step
from slopllm_b200.models.weights import random_model
from slopllm_b200.ops.meta_ops import MetaOps
from slopllm_b200.runtime.planner import padded_kv_len, smallt_splits, sparse_mla_splits
from slopllm_b200.runtime.workspace import UsingHolder, Workspace, walk_tensors


def test_workspace_alloc_free_and_lineage():
    ws = Workspace(1 << 16)
    a = ws.alloc((100,), torch.float32, "a", stream=1)
    b = ws.alloc((64, 4), torch.bfloat16, "b", stream=2)
    assert a.data_ptr() % 256 == 0 and b.data_ptr() % 256 == 0 and a.numel() == 100
    a.fill_(3.0)
    used = ws.used
    ws.free(a)
    # a block freed on stream 1 is reused by stream 1 first, and not handed to another stream before promote()
    c = ws.alloc((100,), torch.float32, "c", stream=2)
    assert c.data_ptr() != a.data_ptr()
    d = ws.alloc((50,), torch.float32, "d", stream=1)
    assert d.data_ptr() == a.data_ptr()
    ws.free(d)
    ws.promote(1)
    assert ws.used < used + 1024
    with pytest.raises(ValueError):
        ws.free(d)
    assert [n for n, _, _ in ws.layout()] == ["b", "c"]


def test_workspace_scope_freeze_reset_and_exhaustion():
    ws = Workspace(4096)
    w = ws.alloc((256,), torch.float32, "weight")
    ws.freeze()
    with ws.scope():
        t1 = ws.alloc((128,), torch.float32, "tmp1")
        t2 = ws.alloc((128,), torch.float32, "tmp2")
        assert len(ws.live) == 3 and t1.data_ptr() != t2.data_ptr()
    assert len(ws.live) == 1
    with pytest.raises(MemoryError):
        ws.alloc((4096,), torch.float32)
    ws.reset()
    assert len(ws.live) == 1 and ws.live[w.data_ptr()].name == "weight"
    big = ws.alloc((700,), torch.float32)             # the lineage blocks were returned to the heap
    assert big.numel() == 700


def test_using_holder_and_tensor_tree():
    log = []

    class D:
        def __init__(self, n):
            self.n = n

        def dispose(self):
            log.append(self.n)

    with UsingHolder(D(1)) as h:
        h.replace(D(2))
        kept = h.detach()
        h.replace(D(3))
    assert log == [1, 3] and kept.n == 2
    seen = []
    walk_tensors({"a": [torch.zeros(1), (torch.ones(2), 5)], "b": type("O", (), {})()}, lambda t: seen.append(t.numel()))
    assert seen == [1, 2]


def test_planner():
    assert sparse_mla_splits(1, 8, 2048) == 32             # one token, one head group: split the 2048 keys 32 ways
    assert sparse_mla_splits(8, 64, 2048) == 9
    assert sparse_mla_splits(4096, 64, 2048) == 1
    assert smallt_splits(8, 2784, 6144) == 8 and smallt_splits(8, 154880 // 8, 6144) == 1
    assert padded_kv_len(5) == 1024 and padded_kv_len(1025) == 2048 and padded_kv_len(4096) == 4096


def test_meta_ops_runs_the_model_without_memory():
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0)
    ops = MetaOps(cfg)
    m = GlmMoeDsaModel(cfg, w, ops=ops)
    cache = KVCacheTensors.allocate(cfg, 4, "cpu")
    T = 37
    st = make_step(list(range(T)), list(range(T)), [0] * T, [[0, 1, 2, 3]])
    hidden = m.forward_hidden(st, cache)
    assert hidden.device.type == "meta" and tuple(hidden.shape) == (T, cfg.hidden_size)
    s = ops.summary()
    assert s["calls"]["linear"] >= 3 * cfg.num_hidden_layers and s["total_flops"] > 0 and s["total_weight_bytes"] > 0
    assert s["calls"]["moe"] == cfg.num_hidden_layers - cfg.first_k_dense_replace


def test_every_called_kernel_entry_point_is_declared_and_exported():
    """Each `N.call("sl_...")` in the package names an entry point with a registered ctypes signature whose arity
    matches the C prototype's parameter count, and the built kernel library exports it."""
    import os
    import re

    import slopllm_b200
    import slopllm_b200.checkpoint.csf_gpu  # noqa: F401  (registers its signature on import or first use)
    import slopllm_b200.ops.cuda_ops  # noqa: F401
    import slopllm_b200.ops.fp4  # noqa: F401
    import slopllm_b200.parallel.ep  # noqa: F401
    import slopllm_b200.parallel.nvlink  # noqa: F401
    from slopllm_b200.ops import native as N
    root = os.path.dirname(slopllm_b200.__file__)
    called = set()
    for d, _, files in os.walk(root):
        for f in files:
            if f.endswith(".py"):
                called |= set(re.findall(r'\.call\(\s*"(sl_\w+)"', open(os.path.join(d, f)).read()))
    assert len(called) > 40
    lazy = {"sl_csf_decode"}                                   # registered by csf_gpu on first use
    assert not [n for n in sorted(called - lazy) if n not in N._SIGS]
    # prototypes in the CUDA sources: SL_API int name(args...)
    protos = {}
    for f in os.listdir(os.path.join(root, "csrc")):
        if f.endswith(".cu"):
            src = open(os.path.join(root, "csrc", f)).read()
            for m in re.finditer(r"SL_API\s+\w[\w\s\*]*?\b(sl_\w+)\s*\(([^)]*)\)", src):
                args = [a for a in m.group(2).split(",") if a.strip() and a.strip() != "void"]
                protos[m.group(1)] = len(args)
    for n in sorted(called - lazy):
        assert n in protos, n
        assert len(N._SIGS[n]) == protos[n], (n, len(N._SIGS[n]), protos[n])
    if os.path.exists(N.KERNELS_SO):
        lib = N.kernels()
        assert not [n for n in sorted(called) if not hasattr(lib, n)]


def test_bulk_allreduce_host_logic(monkeypatch):
    """Host side of the prefill-sized all-reduce on CPU buffers with the kernel calls recorded instead of launched:
    which row counts take the path, lane per stream, pointer tables of the GEMM view and of the collective view, and the
    launch sequence of producer / owner step / consumer."""
    import torch

    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.ops import native as N
    from slopllm_b200.parallel import nvlink as NV
    from slopllm_b200.parallel.dist import ParallelContext
    calls = []
    monkeypatch.setattr(N, "call", lambda name, *a: calls.append((name, a)))
    monkeypatch.setattr(N, "stream", lambda: 0)
    W, H, rows = 4, 1024, 512
    lay = NV.SymmetricRegion.layout(W, 32, H, 0, None, rows)
    assert len(lay["bulk"]) == NV.SymmetricRegion.BULK_LANES
    # areas of one lane and of different lanes do not overlap and are 256-byte aligned
    spans = sorted((off, off + size) for lane in lay["bulk"] for off, size in
                   ((lane["stage"], rows * H * 2), (lane["full"], rows * H * 2), (lane["rs_count"], 4 * rows // 32),
                    (lane["ag_count"], 4 * 8)))
    assert all(a % 256 == 0 for a, _ in spans) and all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1))
    assert spans[-1][1] <= lay["total"]
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8) for _ in range(W)]
    ptrs = [b.data_ptr() for b in bufs]
    regions = [NV.SymmetricRegion(r, W, 32, H, bufs[r], ptrs, bulk_rows=rows) for r in range(W)]
    comm = NV.NvlinkComm(ParallelContext(2, W, torch.device("cpu")), GlmMoeDsaConfig.tiny(), region=regions[2])
    assert comm.partial_sink(16).__class__.__name__ == "PushSink"            # decode-sized: tagged-word path
    assert comm.partial_sink(100) is None and comm.partial_sink(rows * 2) is None and comm.partial_sink(64) is None
    sink = comm.partial_sink(256)
    assert isinstance(sink, NV.BulkSink) and sink.lane == 0
    assert (sink.ctx.rank, sink.ctx.world, sink.ctx.slot_rows, sink.ctx.row_len) == (2, W, 64, H)
    assert (sink.rs.rank, sink.rs.world, sink.rs.slot_rows, sink.rs.row_len) == (2, W, 64, H)
    for r in range(W):
        assert sink.ctx.stage[r] == sink.rs.bufs[r] == ptrs[r] + lay["bulk"][0]["stage"]
        assert sink.ctx.rs_count[r] == sink.rs.flags[r] == ptrs[r] + lay["bulk"][0]["rs_count"]
        assert sink.ctx.full[r] == ptrs[r] + lay["bulk"][0]["full"] and sink.ctx.ag_count[r] == ptrs[r] + lay["bulk"][0]["ag_count"]
    sink.push_tensor(torch.zeros(256, H))
    comm.allreduce_add_rmsnorm(None, sink, None, torch.ones(H, dtype=torch.bfloat16), 1e-5)
    assert [c[0] for c in calls] == ["sl_rs_push_rows", "sl_rs_reduce_ag", "sl_bulk_add_rmsnorm"]
    # without the switch no lanes are laid out and every prefill-sized sum keeps the library path
    plain = NV.SymmetricRegion(0, W, 32, H, torch.zeros(NV.SymmetricRegion.layout(W, 32, H)["total"], dtype=torch.uint8), ptrs)
    assert NV.NvlinkComm(ParallelContext(0, W, torch.device("cpu")), GlmMoeDsaConfig.tiny(), region=plain).partial_sink(256) is None


def test_symmetric_region_guard_zones_detect_overruns():
    import pytest
    import torch

    from slopllm_b200.parallel.nvlink import SymmetricRegion
    W, H = 2, 256
    lay = SymmetricRegion.layout(W, 32, H, 1024, (32, 8, 64), 64)
    assert len(lay["guards"]) >= 8 + 3 + 1 + 2 + 4 * SymmetricRegion.BULK_LANES
    buf = torch.zeros(lay["total"], dtype=torch.uint8)
    rg = SymmetricRegion(0, W, 32, H, buf, [buf.data_ptr()] * W, gather_bytes=1024, cp_shape=(32, 8, 64), bulk_rows=64)
    rg.check_canaries()
    # every area ends where its guard zone begins: a store one byte past the last receive slot lands in a guard
    end_of_data2 = lay["data"][2] + W * 32 * H * 4
    assert end_of_data2 in lay["guards"]
    buf[end_of_data2] = 1
    with pytest.raises(RuntimeError, match="guard zone"):
        rg.check_canaries()
    rg.write_canaries()
    rg.check_canaries()


def test_indexer_score_matrix_is_sized_by_context_and_blocked_by_budget():
    """Rows of queries scored per launch: the whole step while [T, keys] fp32 fits the budget (every decode step, every
    prefill chunk at ordinary context), blocks of a multiple of 8 rows beyond it (reference `tests/test_indexer_sizing.ts`:
    the score matrix must not be sized by the cache capacity)."""
    from slopllm_b200.ops.cuda_ops import CudaOps
    budget = CudaOps.IDX_SCORE_BUDGET
    assert CudaOps.score_rows_per_block(8, 4096) == 8
    assert CudaOps.score_rows_per_block(8192, 16384) == 8192                 # 128K context over 8 CP ranks
    rows = CudaOps.score_rows_per_block(8192, 1 << 20)                       # 1M keys on one rank
    assert rows % 8 == 0 and 8 <= rows < 8192 and rows * (1 << 20) * 4 <= budget
    assert CudaOps.score_rows_per_block(8192, 1 << 28) == 8                  # never below one 8-row tile


def test_runtime_library_exports_what_the_python_side_declares():
    """Every `rt_*` function that `runtime/native_runtime.py` types is defined in the C++ runtime sources and exported by the
    built library."""
    import os
    import re

    import slopllm_b200
    from slopllm_b200.ops import native as N
    root = os.path.dirname(slopllm_b200.__file__)
    declared = set(re.findall(r"lib\.(rt_\w+)", open(os.path.join(root, "runtime", "native_runtime.py")).read()))
    defined = set()
    for f in os.listdir(os.path.join(root, "csrc", "runtime")):
        if f.endswith(".cpp"):
            defined |= set(re.findall(r"RT_API\s+[\w\s\*]*?\b(rt_\w+)\s*\(", open(os.path.join(root, "csrc", "runtime", f)).read()))
    assert len(declared) >= 18 and declared <= defined, sorted(declared - defined)
    if os.path.exists(N.RUNTIME_SO):
        lib = N.runtime()
        assert not [n for n in sorted(declared) if not hasattr(lib, n)]


def test_op_timers_attach_counts_a_collective_once():
    """`OpTimers.attach` times a second object (the communicator) under the same nesting rule: a collective that calls
    a backend op inside is one entry, the op on its own another; `restore` puts both objects back."""
    from slopllm_b200.utils.tracing import OpTimers

    class Ops:
        def combine(self, x):
            return x + 1

    class Comm:
        def __init__(self, ops):
            self.ops = ops

        def cp_merge(self, x):
            return self.ops.combine(x) * 2

    ops = Ops()
    comm = Comm(ops)
    orig_ops, orig_comm = ops.combine.__func__, comm.cp_merge.__func__
    t = OpTimers(ops)
    t.attach(comm, ["cp_merge"], prefix="comm.")
    assert comm.cp_merge(1) == 4 and ops.combine(1) == 2
    if torch.cuda.is_available():
        names = {r["op"]: r["calls"] for r in t.summary()}
        assert names == {"comm.cp_merge": 1, "combine": 1}
    t.restore()
    assert ops.combine.__func__ is orig_ops and comm.cp_merge.__func__ is orig_comm


def test_engine_step_buffers_live_in_the_workspace_arenas():
    """The engine's static step inputs, their host mirrors and the result read-back buffers are carved from its two
    arenas (`runtime/workspace.py`) and frozen; a shape that does not fit falls back to buffers of its own."""
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.runtime import engine as E
    cfg = GlmMoeDsaConfig.tiny()
    eng = E.Engine(cfg, GlmMoeDsaModel(cfg, random_model(cfg, 0)), num_pages=8, max_batch=2, max_seq_len=256, cuda_graph=False)
    buf = eng._buffers(2, 1)
    lo, hi = eng.step_arena.buffer.data_ptr(), eng.step_arena.buffer.data_ptr() + eng.step_arena.nbytes
    assert lo <= buf.dev.data_ptr() < hi
    assert eng.host_arena.buffer.data_ptr() <= buf.host.data_ptr() < eng.host_arena.buffer.data_ptr() + eng.host_arena.nbytes
    assert buf.dev.data_ptr() in eng.step_arena.frozen and int(buf.dev.abs().sum()) == 0
    names = [n for n, _, _ in eng.step_arena.layout()]
    assert "step_dev_2x1" in names
    s = eng.kv.new_sequence()
    last, _ = eng.prefill([s], [[1, 2, 3, 4, 5]], chunk_size=64)
    eng.decode_step([s], last)
    assert any(n.startswith("result_") for n, _, _ in eng.host_arena.layout())
    big = E.StepBuffers.create(64, 4, 1 << 20, eng.device, eng.host_arena, eng.step_arena)      # larger than the arena
    assert not (lo <= big.dev.data_ptr() < hi)
