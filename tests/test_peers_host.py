"""Host logic of the peer-buffer setup, no GPU: two ranks run as threads against a stand-in
library; a rank whose allocation or mapping fails must make both ranks fail together (nobody is
left waiting in a host collective), and the healthy path must fill the pointer table."""
import threading

import pytest


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


class FakeLib:
    def __init__(self, rank, fail_alloc=False, fail_open=False):
        self.rank, self.fail_alloc, self.fail_open = rank, fail_alloc, fail_open
        self.next = 0x1000 * (rank + 1)

    def h3x_peer_alloc(self, handle, nbytes, out):
        if self.fail_alloc:
            return 0
        self.next += 0x100
        out[0] = self.rank + 1          # the "handle" names its owner
        out[1] = self.next & 0xff
        return self.next

    def h3x_peer_open(self, handle, blob):
        return 0 if self.fail_open else 0x90000 + blob[0] * 0x100 + blob[1]

    def h3x_tensor_wrap(self, handle, ptr, elements, dtype):
        return ptr

    def h3x_peer_close(self, handle, ptr):
        return 1

    def h3x_peer_free(self, handle, ptr):
        return 1


class FakeGpu:
    def __init__(self, lib):
        self.lib, self.handle = lib, 1

    def error(self):
        return "stand-in failure"

    def wrap(self, ptr, elements, dtype):
        return ("tensor", ptr, elements)


def run_two_ranks(pkg, **faults):
    barrier = threading.Barrier(2)
    slots, results = [None, None], [None, None]

    def gather_for(rank):
        def gather(obj):
            slots[rank] = obj
            barrier.wait(timeout=10)
            out = list(slots)
            barrier.wait(timeout=10)
            return out
        return gather

    def work(rank):
        lib = FakeLib(rank, fail_alloc=faults.get("fail_alloc") == rank, fail_open=faults.get("fail_open") == rank)
        ex = pkg.PeerExchange(FakeGpu(lib), 2, rank, gather_for(rank))
        try:
            local = ex.setup(rows_local=4, heads=2, head_dim=128)
            results[rank] = ("ok", ex, local)
        except pkg.H3Error as err:
            results[rank] = ("error", str(err))

    threads = [threading.Thread(target=work, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
        assert not t.is_alive(), "a rank is stuck in a host collective"
    return results


def test_healthy_setup_fills_the_table(pkg):
    (s0, ex0, local0), (s1, ex1, _) = run_two_ranks(pkg)
    assert s0 == s1 == "ok"
    assert ex0.peers.world == 2 and ex0.peers.rank == 0 and ex0.peers.rows_local == 4
    for name in ("q", "k", "v", "o", "flags"):
        mine, theirs = getattr(ex0.peers, name)[0], getattr(ex0.peers, name)[1]
        assert mine and theirs and mine != theirs
        assert getattr(ex1.peers, name)[1] and getattr(ex1.peers, name)[0]
    assert local0["q"][1] == ex0.peers.q[0]              # the local tensor wraps this rank's block


@pytest.mark.parametrize("fault", [{"fail_alloc": 1}, {"fail_open": 0}])
def test_a_failing_rank_fails_both(pkg, fault):
    r0, r1 = run_two_ranks(pkg, **fault)
    assert r0[0] == r1[0] == "error"
    assert "unavailable" in r0[1] and "unavailable" in r1[1]
