"""Host-side logic of the FSDP all-gather communicator (ring of output buffers, fall-backs),
with the symmetric workspaces replaced by plain CPU buffers."""
import pytest
import torch

from dion_b200.parallel import fsdp_comm


class _FakeBuf:
    def __init__(self, nbytes):
        self.local = torch.zeros(nbytes, dtype=torch.uint8)


class _FakeRing:
    def __init__(self, nbytes):
        self.buf = _FakeBuf(nbytes)
        self.capacity = nbytes
        self.gathers = []

    def view(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buf.local[:nbytes].view(dtype).view(tuple(shape))

    def all_gather_(self, slot):
        self.gathers.append(slot)


def _make(num=3, nbytes=4096, world=2, rank=1):
    comm = object.__new__(fsdp_comm.SymmetricAllGather)
    comm.group, comm.device = None, torch.device("cpu")
    comm.world, comm.rank, comm.max_bytes = world, rank, nbytes
    comm.rings = [_FakeRing(nbytes) for _ in range(num)]
    comm._by_ptr = {r.view((1,), torch.uint8).data_ptr(): r for r in comm.rings}
    comm._idle_users = [fsdp_comm._storage_users(r.buf.local) for r in comm.rings]
    comm._next, comm.calls, comm.fallbacks = 0, 0, 0
    return comm


def test_ring_hands_out_buffers_in_order_and_detects_reuse_while_referenced():
    comm = _make(num=2)
    a = comm.allocate((256,), dtype=torch.float32, device=torch.device("cpu"))
    b = comm.allocate((256,), dtype=torch.float32, device=torch.device("cpu"))
    assert a.data_ptr() == comm.rings[0].buf.local.data_ptr()
    assert b.data_ptr() == comm.rings[1].buf.local.data_ptr()
    with pytest.raises(RuntimeError, match="still referenced"):
        comm.allocate((256,), dtype=torch.float32, device=torch.device("cpu"))   # `a` is alive
    comm._next -= 1
    part = a[:16]          # a derived view keeps the buffer busy even when `a` itself is gone
    del a
    with pytest.raises(RuntimeError):
        comm.allocate((256,), dtype=torch.float32, device=torch.device("cpu"))
    comm._next -= 1
    del part
    c = comm.allocate((256,), dtype=torch.float32, device=torch.device("cpu"))
    assert c.data_ptr() == comm.rings[0].buf.local.data_ptr()


def test_oversized_requests_get_ordinary_memory():
    comm = _make(nbytes=1024)
    t = comm.allocate((1024,), dtype=torch.float32, device=torch.device("cpu"))
    assert t.data_ptr() not in comm._by_ptr and comm._next == 0


def test_in_place_gather_launches_on_the_owning_ring():
    comm = _make(world=2, rank=1)
    out = comm.allocate((64,), dtype=torch.float32, device=torch.device("cpu"))
    inp = out[32:]                      # FSDP's copy-in leaves the shard at the rank's slot
    assert comm(out, inp, None) is None
    assert comm.rings[0].gathers == [32 * 4] and comm.calls == 1
    # a shard that lies elsewhere is copied into its slot first
    out2 = comm.allocate((64,), dtype=torch.float32, device=torch.device("cpu"))
    comm(out2, torch.full((32,), 7.0), None)
    assert torch.all(out2[32:] == 7.0) and comm.rings[1].gathers == [128]


def test_all_reduce_slices_partition_the_buffer():
    """Each rank reduces one slice of 16-byte vectors; over all ranks the slices cover the data
    exactly once, for sizes that do not divide evenly too (host arithmetic of
    ``SymmetricAllReduce.all_reduce_`` / ``all_gather_``, no GPU needed)."""
    import torch
    from dion_b200.parallel.symm import SymmetricAllReduce
    for world in (2, 3, 4, 8):
        for numel, dtype in ((1, torch.float32), (5, torch.bfloat16), (4096, torch.float32),
                             (1000003, torch.bfloat16), (7 * world * 4, torch.float32)):
            covered = []
            for rank in range(world):
                red = object.__new__(SymmetricAllReduce)
                red.world, red.rank, red.capacity = world, rank, 1 << 30
                calls = []
                red._launch = lambda b, e, dt, sc, gather, calls=calls: calls.append((b, e, dt, sc, gather))
                red.all_reduce_(numel, dtype, op="avg")
                (b, e, dt, sc, gather), = calls
                assert dt == (0 if dtype == torch.float32 else 1) and not gather
                assert abs(sc - 1.0 / world) < 1e-12
                covered.append((b, max(b, e)))
            esize = 4 if dtype == torch.float32 else 2
            nvec = (numel * esize + 15) // 16
            pos = 0
            for b, e in covered:            # ranks in order: contiguous, disjoint, complete
                assert b == min(pos, b) or b >= pos
                if e > b:
                    assert b == pos
                    pos = e
            assert pos == nvec
    red = object.__new__(SymmetricAllReduce)
    red.world, red.rank, red.capacity = 4, 2, 1 << 20
    calls = []
    red._launch = lambda b, e, dt, sc, gather: calls.append((b, e, gather))
    red.all_gather_(4096)
    assert calls == [(2 * 256, 3 * 256, True)]
    import pytest
    with pytest.raises(ValueError):
        red.all_gather_(24)                 # slots are whole 16-byte vectors
    with pytest.raises(ValueError):
        red.all_gather_(1 << 20)            # world * slot must fit
