"""Host API of the symmetric-heap context on the CPU back end (single process).

Covers what ``iris/iris.py:96-314`` promises: bump allocation with 1024-byte alignment, ``MemoryError`` on
exhaustion, the torch-like factories and their defaults, ``out=`` validation, logging prefix.
"""
import pytest
import torch

import iris_b200 as iris


@pytest.fixture()
def ctx():
    c = iris.iris(1 << 20, backend="cpu")
    yield c
    c.close()


def test_ranks_and_bases(ctx):
    assert ctx.get_rank() == 0 and ctx.get_num_ranks() == 1
    hb = ctx.get_heap_bases()
    assert hb.dtype == torch.uint64 and hb.numel() == 1
    assert int(hb[0]) == ctx.heap_base()
    assert ctx.get_device() == torch.device("cpu")
    assert ctx.wall_clock_rate(0) == 1_000_000
    assert ctx.get_cu_count() >= 1


def test_alignment_and_exhaustion(ctx):
    a = ctx.allocate(3, torch.float32)
    b = ctx.allocate(1, torch.int8)
    assert (b.data_ptr() - a.data_ptr()) == 1024
    assert a.data_ptr() % 1024 == ctx.heap_base() % 1024
    with pytest.raises(MemoryError, match="Heap out of memory"):
        ctx.allocate(1 << 20, torch.int8)


def test_factories_defaults(ctx):
    z = ctx.zeros(4, 5)
    assert z.dtype == torch.int32 and z.shape == (4, 5) and int(z.sum()) == 0
    z2 = ctx.zeros((2, 3), dtype=torch.float32)
    assert z2.shape == (2, 3)
    o = ctx.ones(7)
    assert o.dtype == torch.get_default_dtype() and float(o.sum()) == 7
    f = ctx.full((2, 2), 5)
    assert f.dtype == torch.int32 and int(f.sum()) == 20
    e = ctx.empty((3,), dtype=torch.float16)
    assert e.dtype == torch.float16 and e.numel() == 3
    u = ctx.uniform((100,), low=2.0, high=3.0)
    assert float(u.min()) >= 2.0 and float(u.max()) <= 3.0
    r = ctx.randint((50,), 0, 4)
    assert r.dtype == torch.int32 and int(r.max()) < 4
    ar = ctx.arange(5)
    assert ar.dtype == torch.int64 and ar.tolist() == [0, 1, 2, 3, 4]
    arf = ctx.arange(0.0, 1.0, 0.25)
    assert arf.dtype == torch.get_default_dtype() and arf.numel() == 4
    ls = ctx.linspace(0, 1, 5)
    assert ls.tolist() == pytest.approx([0, 0.25, 0.5, 0.75, 1.0])
    zl = ctx.zeros_like(torch.ones(2, 3))
    assert zl.shape == (6,)
    for t in (z, o, f, e, u, r, ar, ls, zl):
        assert ctx.on_heap(t)


def test_randn_is_seed_deterministic(ctx):
    torch.manual_seed(123)
    a = ctx.randn(16, 4, dtype=torch.float32)
    torch.manual_seed(123)
    b = torch.randn(64, dtype=torch.float32).reshape(16, 4)
    assert torch.equal(a, b)


def test_out_validation(ctx):
    buf = ctx.zeros(8, dtype=torch.float32)
    ctx.ones(8, out=buf, dtype=torch.float32)
    assert float(buf.sum()) == 8
    with pytest.raises(RuntimeError, match="elements"):
        ctx.ones(4, out=buf, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="dtype"):
        ctx.ones(8, out=buf, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="symmetric heap"):
        ctx.ones(8, out=torch.zeros(8), dtype=torch.float32)


def test_logging_prefix(ctx, capsys):
    ctx.log("hello")
    assert "[Iris] [0/1] hello" in capsys.readouterr().out


def test_broadcast_and_barrier_single(ctx):
    assert ctx.broadcast(3.5, 0) == 3.5
    ctx.barrier()


def test_translate_host_mirror():
    assert iris.translate(1100, 0, 1, [1000, 5000]) == 5100


def test_local_world_cpu_rma_all_ops():
    ranks = iris.Iris.local_world(3, heap_size=1 << 16, backend="cpu")
    bufs = [c.ones(32, dtype=torch.float32) for c in ranks]
    outs = [c.zeros(32, dtype=torch.float32) for c in ranks]
    # load from every rank and sum: world * 1 (tests/unittests/test_load.py:69-70)
    for c, b, o in zip(ranks, bufs, outs):
        iris.load(c, b, o)
    assert all(torch.equal(o, torch.full((32,), 3.0)) for o in outs)
    # atomic_add of 1 from every rank to every rank: 1 + world (tests/unittests/test_atomic_add.py)
    for c, b in zip(ranks, bufs):
        iris.atomic_add(c, b, 1.0, sem="release", scope="sys")
    assert all(torch.equal(b, torch.full((32,), 4.0)) for b in bufs)
    # cas 0 -> world on int64 (tests/unittests/test_atomic_cas.py)
    flags = [c.zeros(1, dtype=torch.int64) for c in ranks]
    for c, f in zip(ranks, flags):
        iris.atomic_cas(c, f, 0, 3, sem="acq_rel", scope="sys")
    assert all(int(f[0]) == 3 for f in flags)
    # xchg
    xs = [c.zeros(4, dtype=torch.int32) for c in ranks]
    olds = [c.full((4,), -1, dtype=torch.int32) for c in ranks]
    for c, x, o in zip(ranks, xs, olds):
        iris.atomic_xchg(c, x, 7, old=o)
    assert all(x.tolist() == [7] * 4 for x in xs)
    # put local -> every rank
    srcs = [c.full((8,), r + 1, dtype=torch.int8) for r, c in enumerate(ranks)]
    dsts = [c.zeros(8, dtype=torch.int8) for c in ranks]
    iris.put(ranks[2], srcs[2], dsts[2])
    assert all(d.tolist() == [3] * 8 for d in dsts)


def test_unsupported_pairs_raise():
    (c,) = iris.Iris.local_world(1, heap_size=1 << 16, backend="cpu")
    b = c.zeros(4, dtype=torch.int8)
    with pytest.raises(TypeError):
        iris.atomic_add(c, b, 1)


def test_debug_heap_guards_and_reset():
    """Guard bytes behind every allocation: an overrun is reported at the next barrier with the allocation it
    belongs to; ``reset`` forgets the allocations above the mark; a clean heap passes."""
    from iris_b200.context import IrisHeapCorruption
    ranks = iris.Iris.local_world(2, heap_size=1 << 20, backend="cpu", debug_heap=True)
    c = ranks[0]
    a = [r.zeros(100, dtype=torch.int32) for r in ranks]
    mark = c.mark()
    b = [r.ones(33, dtype=torch.float32) for r in ranks]
    for r in ranks:
        r.barrier()                                   # clean
    assert c.allocation_digest() == ranks[1].allocation_digest() and c.allocation_digest()[0] == 3
    # 132 bytes were asked for; the 16-byte round-up is tolerated, byte 144 is guarded
    c.memory_pool[c.offset_of(b[0]) + 143] = 7
    c.barrier()
    c.memory_pool[c.offset_of(b[0]) + 144] = 7
    with pytest.raises(IrisHeapCorruption, match=r"allocation #2 \(132 bytes of torch.float32"):
        c.barrier()
    c.reset(mark)
    ranks[1].reset(mark)
    c.barrier()                                       # the overrun allocation is gone
    assert c.allocation_digest()[0] == 2
    a[0].fill_(5)                                     # writing inside an allocation never trips a guard
    c.barrier()
    ranks[0].close()


def test_debug_heap_divergence_in_a_local_world():
    from iris_b200.context import IrisDivergenceError
    ranks = iris.Iris.local_world(2, heap_size=1 << 20, backend="cpu", debug_heap=True)
    ranks[0].zeros(10)
    ranks[1].zeros(11)
    with pytest.raises(IrisDivergenceError):
        ranks[0].barrier()
    ranks[0].close()


def test_log_levels(ctx, capsys):
    from iris_b200 import context as C
    saved = (C.STATS, C.LOGGING, C.DEBUG)
    try:
        C.set_log_level("quiet")
        ctx.log("a"), ctx.log_stats("b"), ctx.log_debug("c")
        assert capsys.readouterr().out == ""
        C.set_log_level("stats")
        ctx.log("a"), ctx.log_stats("b"), ctx.log_debug("c")
        assert capsys.readouterr().out.strip().endswith("b")
        C.set_log_level("debug")
        ctx.log("a"), ctx.log_stats("b"), ctx.log_debug("c")
        assert [ln[-1] for ln in capsys.readouterr().out.strip().splitlines()] == ["a", "b", "c"]
        with pytest.raises(ValueError):
            C.set_log_level("loud")
    finally:
        C.STATS, C.LOGGING, C.DEBUG = saved
