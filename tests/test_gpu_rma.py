"""Device RMA API on the GPU with the reference's unit-test semantics and parametrisation
(``tests/unittests/test_load.py:34-51``, ``test_atomic_add.py:31-65``, ``test_atomic_cas.py:26-49``,
``test_atomic_xchg.py:25-48``) plus the ``relaxed`` semantics the reference never tests.  Ranks are simulated
in one process on one GPU; these kernels do not wait on one another, so one launch per rank is fine."""
import pytest
import torch

import iris_b200 as iris
from iris_b200.ops import p2p

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

WORLD = 4
SEMS = ["relaxed", "acquire", "release", "acq_rel"]
SCOPES = ["cta", "gpu", "sys"]


@pytest.fixture(scope="module")
def ranks():
    r = iris.Iris.local_world(WORLD, heap_size=256 << 20)
    yield r
    r[0].close()


@pytest.fixture(autouse=True)
def _rewind(ranks):
    for c in ranks:
        c.reset()
    yield


@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block", [1, 8, 16, 32])
def test_load_store_get_put(ranks, dtype, block):
    data = [c.ones(block, dtype=dtype) for c in ranks]
    res = [c.zeros(block, dtype=dtype) for c in ranks]
    tmp = [c.zeros(block, dtype=dtype) for c in ranks]
    dst = [c.zeros(block, dtype=dtype) for c in ranks]
    dst2 = [c.zeros(block, dtype=dtype) for c in ranks]
    for i, c in enumerate(ranks):
        iris.load(c, data[i], res[i], block=block)
    torch.cuda.synchronize()
    for r in res:
        torch.testing.assert_close(r, torch.full_like(r, WORLD), rtol=0, atol=0)
    for i, c in enumerate(ranks):
        res[i].zero_()
        iris.get(c, data[i], tmp[i], res[i], block=block)
        iris.store(c, dst[i], 1, block=block)
        iris.put(c, data[i], dst2[i], block=block)
    torch.cuda.synchronize()
    for i in range(WORLD):
        torch.testing.assert_close(res[i], torch.full_like(res[i], WORLD), rtol=0, atol=0)
        torch.testing.assert_close(dst[i], torch.ones_like(dst[i]), rtol=0, atol=0)
        torch.testing.assert_close(dst2[i], torch.ones_like(dst2[i]), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64, torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("scope", SCOPES)
def test_atomic_add(ranks, dtype, sem, scope):
    for block in (1, 8, 16, 32):
        acc = [c.zeros(block, dtype=dtype) for c in ranks]
        for i, c in enumerate(ranks):
            iris.atomic_add(c, acc[i], 1, sem=sem, scope=scope, block=block)
        torch.cuda.synchronize()
        for a in acc:
            torch.testing.assert_close(a, torch.full_like(a, WORLD), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64, torch.float32])
def test_atomic_sub_returns_old(ranks, dtype):
    c = ranks[0]
    buf = c.full((8,), 10, dtype=dtype)
    old = c.zeros(8, dtype=dtype)
    iris.atomic_sub(c, buf, 3, old=old, target=0)
    torch.cuda.synchronize()
    assert buf.tolist() == [7] * 8 and old.tolist() == [10] * 8


@pytest.mark.parametrize("dtype", [torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("scope", SCOPES)
def test_atomic_cas(ranks, dtype, sem, scope):
    f = [c.zeros(1, dtype=dtype) for c in ranks]
    for i, c in enumerate(ranks):
        iris.atomic_cas(c, f[i], 0, WORLD, sem=sem, scope=scope, block=1)
    torch.cuda.synchronize()
    assert all(int(x[0]) == WORLD for x in f)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64, torch.float32])
@pytest.mark.parametrize("sem", SEMS)
@pytest.mark.parametrize("scope", SCOPES)
def test_atomic_xchg(ranks, dtype, sem, scope):
    x = [c.zeros(1, dtype=dtype) for c in ranks]
    for i, c in enumerate(ranks):
        iris.atomic_xchg(c, x[i], WORLD, sem=sem, scope=scope, block=1)
    torch.cuda.synchronize()
    assert all(int(v[0]) == WORLD for v in x)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_bandwidth_kernels_values(ranks, dtype):
    n = (1 << 20) // torch.empty((), dtype=dtype).element_size()
    src = [c.full((n,), r + 1, dtype=dtype) for r, c in enumerate(ranks)]
    out = [c.zeros(n, dtype=dtype) for c in ranks]
    words = [c.zeros(n * src[0].element_size() // 4, dtype=torch.int32) for c in ranks]
    c0 = ranks[0]
    p2p.load(c0, src[0], out[0], target=2)
    torch.cuda.synchronize()
    assert torch.equal(out[0], torch.full_like(out[0], 3))
    p2p.all_load(c0, src[0], out[0])
    torch.cuda.synchronize()
    assert torch.equal(out[0], torch.full_like(out[0], sum(range(1, WORLD + 1))))
    p2p.store(c0, words[0], target=1)
    torch.cuda.synchronize()
    expect = torch.arange(words[0].numel(), dtype=torch.int32, device="cuda")
    assert torch.equal(words[1], expect) and int(words[0].abs().sum()) == 0
    p2p.all_store(ranks[3], words[3])
    torch.cuda.synchronize()
    assert all(torch.equal(words[r], expect) for r in (0, 1, 2)) and int(words[3].abs().sum()) == 0


def test_atomic_bandwidth_kernels(ranks):
    n = 1 << 16
    f = [c.zeros(n, dtype=torch.float32) for c in ranks]
    x = [c.zeros(n, dtype=torch.int32) for c in ranks]
    old = [c.full((n,), -1, dtype=torch.int32) for c in ranks]
    p2p.atomic_add_f32(ranks[0], f[0], target=1)
    p2p.atomic_add_f32(ranks[0], f[0], target=1, vec4=True)
    p2p.atomic_xchg_i32(ranks[2], x[2], old[2], target=3)
    torch.cuda.synchronize()
    assert torch.equal(f[1], torch.full_like(f[1], 2)) and float(f[0].sum()) == 0
    assert torch.equal(x[3], torch.ones_like(x[3])) and int(old[2].abs().sum()) == 0


def test_memset_tensor(ranks):
    t = ranks[0].full((1000,), 5, dtype=torch.int32)
    iris.memset_tensor(t, 0)
    torch.cuda.synchronize()
    assert int(t.abs().sum()) == 0
    with pytest.raises(AssertionError):
        iris.memset_tensor(t.float(), 0)


@pytest.mark.parametrize("use_put", [True, False])
def test_message_passing_one_launch(ranks, use_put):
    two = ranks[:2]
    mp = [p2p.MessagePassing(c, nchunks=8, chunk_bytes=1 << 20) for c in two]   # 1 MB chunks
    for epoch in (1, 2):
        mp[0].src.copy_(torch.arange(mp[0].src.numel(), device="cuda", dtype=torch.float32) % 1000 + epoch)
        mp[1].out.zero_()
        for m in mp:
            m.epoch = epoch
        mp[0].run(roles=3, use_put=use_put, advance=False)   # producer and consumer blocks in one cooperative launch
        torch.cuda.synchronize()
        two[1].check_status()
        assert torch.equal(mp[1].out, 2 * mp[0].src), f"epoch {epoch}"


def test_message_passing_replays_from_a_cuda_graph(ranks):
    """device_epoch=True: both sides count their calls in device memory, the launch has no per-call argument, and a
    captured hand-off replays with new data (ordinary calls before and after)."""
    two = ranks[:2]
    mp = [p2p.MessagePassing(c, nchunks=8, chunk_bytes=1 << 18, device_epoch=True, blocks=16) for c in two]

    def fill(seed):
        mp[0].src.copy_(torch.arange(mp[0].src.numel(), device="cuda", dtype=torch.float32) % 997 + seed)

    def check():
        torch.cuda.synchronize()
        two[1].check_status()
        assert torch.equal(mp[1].out, 2 * mp[0].src)

    fill(1)
    mp[0].run(roles=3)
    check()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        mp[0].run(roles=3)
    for i in range(3):
        fill(10 + i)
        mp[1].out.zero_()
        graph.replay()
        check()
    fill(50)
    mp[0].run(roles=3)
    check()
    n = mp[0].nchunks
    assert int(mp[0].arrive[n]) == 5 and int(mp[1].flags[n]) == 5      # calls counted on both sides
    assert int(mp[0].arrive[n + 1]) == 0 and int(mp[1].flags[n + 1]) == 0


def test_bounded_wait_reports_timeout(ranks):
    """A flag that nothing sets: the consumer's wait runs out after 1 ms, the kernel returns normally and the
    host reads a time-out status; the context stays usable."""
    c = ranks[1]
    mp = p2p.MessagePassing(c, nchunks=2, chunk_bytes=4096, producer=0, consumer=1, timeout_ms=1.0)
    mp.run(roles=2)
    torch.cuda.synchronize()
    with pytest.raises(iris.IrisTimeoutError):
        c.check_status()
    c.check_status()  # cleared
    t = c.ones(4, dtype=torch.float32)
    assert float(t.sum()) == 4.0
