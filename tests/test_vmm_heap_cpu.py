"""Orchestration of the CUDA-VMM heap and its NVLS multicast binding (iris_b200/parallel/vmm_heap.py) against a fake
of the native runtime, with the ranks as threads: the order of driver calls, the contiguous mapping, and that a step
failing on ONE rank makes EVERY rank fall back to plain peer access and release what it had created.  The real calls
run in tests/test_gpu_multi.py::test_vmm_heap on two or more GPUs."""
import threading
from types import SimpleNamespace

import pytest

from iris_b200 import _native
from iris_b200.parallel import vmm_heap


class ThreadComm:
    """allgather / broadcast / barrier between the threads of one test."""

    def __init__(self, world):
        self.world = world
        self._bar = threading.Barrier(world)
        self._slots = [None] * world
        self._box = [None]

    def view(self, rank):
        c = self

        class V:
            def allgather_bytes(self, payload):
                c._slots[rank] = bytes(payload)
                c._bar.wait()
                out = list(c._slots)
                c._bar.wait()
                return out

            def broadcast_object(self, obj, root):
                if rank == root:
                    c._box[0] = obj
                c._bar.wait()
                out = c._box[0]
                c._bar.wait()
                return out

            def barrier(self, timeout_s=None):
                c._bar.wait()
        return V()


class FakeRuntime:
    """Records the calls of one rank; descriptors and sockets are numbers in a mailbox shared by all ranks."""
    GRAN = 2 << 20

    def __init__(self, rank, shared, fail=None):
        self.rank, self.shared, self.fail, self.calls, self.error = rank, shared, fail or {}, [], b""

    def _rc(self, name):
        self.calls.append(name)
        if self.fail.get(name) == self.rank:
            self.error = f"{name} refused".encode()
            return 1
        return 0

    def iris_rt_last_error(self):
        return self.error

    def iris_rt_vmm_supported(self, dev):
        return 1

    def iris_rt_vmm_granularity(self, dev):
        return self.GRAN

    def iris_rt_multicast_supported(self, dev):
        return 1

    def iris_rt_multicast_granularity(self, world, size):
        return self.GRAN

    def iris_rt_vmm_create(self, dev, size, handle, fd):
        handle._obj.value, fd._obj.value = 1000 + self.rank, 100 + self.rank
        return self._rc("vmm_create")

    def iris_rt_vmm_reserve(self, size, align, va):
        with self.shared["lock"]:
            self.shared["next_va"] += 1 << 40
            va._obj.value = self.shared["next_va"]
        return self._rc("vmm_reserve")

    def iris_rt_vmm_import(self, fd, handle):
        handle._obj.value = 5000 + fd
        return self._rc("vmm_import")

    def iris_rt_vmm_map(self, va, size, handle, dev):
        self.shared["maps"].append((self.rank, va, size, handle))
        return self._rc("vmm_map")

    def iris_rt_vmm_unmap(self, va, size):
        return self._rc("vmm_unmap")

    def iris_rt_vmm_release(self, handle):
        return self._rc("vmm_release")

    def iris_rt_vmm_address_free(self, va, size):
        return self._rc("vmm_address_free")

    def iris_rt_memset(self, p, v, n):
        return self._rc("memset")

    def iris_rt_multicast_create(self, world, size, handle, fd):
        handle._obj.value, fd._obj.value = 9000, 900
        return self._rc("multicast_create")

    def iris_rt_multicast_add_device(self, handle, dev):
        return self._rc("multicast_add_device")

    def iris_rt_multicast_bind(self, mc, mem, size):
        return self._rc("multicast_bind")

    def iris_rt_multicast_unbind(self, mc, dev, size):
        return self._rc("multicast_unbind")

    # descriptor exchange: a mailbox per socket name
    def iris_rt_fd_listen(self, name):
        with self.shared["lock"]:
            self.shared["boxes"].setdefault(name, [])
            self.shared["socks"].append(name)
            return len(self.shared["socks"]) - 1

    def iris_rt_fd_send(self, name, fd, tag):
        with self.shared["lock"]:
            self.shared["boxes"][name].append((fd, tag))
        return 0

    def iris_rt_fd_recv(self, sock, timeout_ms, tag):
        import time
        name = self.shared["socks"][sock]
        t0 = time.time()
        while time.time() - t0 < timeout_ms / 1e3:
            with self.shared["lock"]:
                if self.shared["boxes"][name]:
                    fd, tg = self.shared["boxes"][name].pop(0)
                    tag._obj.value = tg
                    return fd
            time.sleep(0.001)
        return -1

    def iris_rt_fd_close(self, fd):
        return 0


def _run_world(monkeypatch, world, nvls, fail=None):
    shared = {"lock": threading.Lock(), "next_va": 0, "maps": [], "boxes": {}, "socks": []}
    comm = ThreadComm(world)
    fakes = [FakeRuntime(r, shared, fail) for r in range(world)]
    by_thread = {}
    monkeypatch.setattr(_native, "runtime", lambda: by_thread[threading.get_ident()])
    monkeypatch.setattr(_native, "rt_check", lambda rc, what: (_ for _ in ()).throw(RuntimeError(what)) if rc else None)
    monkeypatch.setenv("IRIS_NVLS", "1" if nvls else "0")
    heaps, logs, errors = [None] * world, [[] for _ in range(world)], []

    def body(rank):
        by_thread[threading.get_ident()] = fakes[rank]
        ctx = SimpleNamespace(gpu_id=rank, cur_rank=rank, num_ranks=world, heap_size=(3 << 20) + 5,
                              comm=comm.view(rank), log=logs[rank].append)
        try:
            heaps[rank] = vmm_heap.create(ctx)
        except Exception as e:  # noqa: BLE001 - reported by the test
            errors.append((rank, repr(e)))
            comm._bar.abort()
    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
    assert not errors, errors
    return heaps, fakes, logs, shared


def test_heaps_are_mapped_contiguously_and_bound(monkeypatch):
    world = 3
    heaps, fakes, logs, shared = _run_world(monkeypatch, world, nvls=True)
    stride = 4 << 20                                     # heap size rounded up to the 2 MB granularity
    for r, h in enumerate(heaps):
        assert h.stride == stride
        assert h.peer_ptrs == [h._va + q * stride for q in range(world)] and h.own_ptr == h.peer_ptrs[r]
        assert h.mc_ptr and h.mc_ptr == h._mc_va and h._mc_bound
        mine = [m for m in shared["maps"] if m[0] == r]
        assert [m[1] for m in mine[:world]] == h.peer_ptrs          # every rank's heap, in rank order
        assert mine[world][3] == (9000 if r == 0 else 5900)         # then the multicast object (imported by fd)
        order = [c for c in fakes[r].calls if c.startswith("multicast")]
        assert order == (["multicast_create"] if r == 0 else []) + ["multicast_add_device", "multicast_bind"]
        assert not logs[r]
    monkeypatch.setattr(_native, "runtime", lambda: fakes[0])   # close() runs on this thread
    heaps[0].close()
    assert fakes[0].calls.count("vmm_unmap") == world + 1 and "multicast_unbind" in fakes[0].calls


@pytest.mark.parametrize("step", ["multicast_create", "multicast_add_device", "multicast_bind", "vmm_map"])
def test_a_failing_step_on_one_rank_makes_every_rank_fall_back(monkeypatch, step):
    world = 3
    failing_rank = 0 if step == "multicast_create" else 1
    fail = {step: failing_rank}
    if step == "vmm_map":          # only the map of the multicast object shall fail: arm it after the heap maps
        fail = {}
    if step == "vmm_map":
        orig = FakeRuntime.iris_rt_vmm_map

        def failing_map(self, va, size, handle, dev):
            rc = orig(self, va, size, handle, dev)
            if self.rank == failing_rank and handle in (9000, 5900):
                self.error = b"vmm_map refused"
                return 1
            return rc
        monkeypatch.setattr(FakeRuntime, "iris_rt_vmm_map", failing_map)
    heaps, fakes, logs, shared = _run_world(monkeypatch, world, nvls=True, fail=fail)
    for r, h in enumerate(heaps):
        assert h.mc_ptr == 0 and h._mc_va == 0 and h._mc_handle == 0 and not h._mc_bound    # nobody keeps a binding
        assert h.peer_ptrs and h.own_ptr == h.peer_ptrs[r]                                    # the heap itself stands
        assert len(logs[r]) == 1 and f"rank(s) [{failing_rank}]" in logs[r][0], logs[r]
        if step in ("multicast_bind", "vmm_map") and not (step == "multicast_bind" and r == failing_rank):
            assert "multicast_unbind" in fakes[r].calls          # what was bound is unbound again


def test_without_nvls_nothing_multicast_is_called(monkeypatch):
    heaps, fakes, logs, _ = _run_world(monkeypatch, 2, nvls=False)
    assert all(h.mc_ptr == 0 for h in heaps)
    assert not any(c.startswith("multicast") for f in fakes for c in f.calls)
