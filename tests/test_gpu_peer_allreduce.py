"""The plugin's push all-reduce on one GPU: the single-rank case, argument checking, and the
bounded wait (a peer that never signals must end in a status word and DEVICE_LOST, with the
tensor untouched and the context still usable).  The two-rank path runs in test_gpu_tp.py."""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu


def test_single_rank_is_identity(ctx):
    v = (np.arange(4096, dtype=np.float32) / 7 - 200).astype(np.float16)
    buf = ctx.upload(v)
    comm, handle = ctx.peer_comm_create(0, 1, v.nbytes)
    try:
        assert len(handle) == B.PEER_HANDLE_BYTES
        for _ in range(5):                                   # epochs 1..5: both parities
            ctx.peer_allreduce(comm, buf, v.size, B.F16)
        assert np.array_equal(buf.to_host(np.float16, v.shape), v)
    finally:
        ctx.peer_comm_destroy(comm)


def test_argument_checks(ctx):
    v = np.zeros(64, np.float16)
    buf = ctx.upload(v)
    comm, _ = ctx.peer_comm_create(0, 1, 128)
    try:
        with pytest.raises(B.BackendError) as e:
            ctx.peer_allreduce(comm, buf, 60, B.F16)          # not a multiple of 8 elements
        assert e.value.code == B.NOT_SUPPORTED
        with pytest.raises(B.BackendError) as e:
            ctx.peer_allreduce(comm, buf, 128, B.F16)         # larger than the window slot / the buffer
        assert e.value.code == B.INVALID_ARGUMENT
        with pytest.raises(B.BackendError) as e:
            ctx.peer_allreduce(comm, buf, 64, B.F32)
        assert e.value.code == B.NOT_SUPPORTED
    finally:
        ctx.peer_comm_destroy(comm)
    with pytest.raises(B.BackendError):
        ctx.peer_comm_create(3, 2, 128)                       # rank outside the world


def test_peer_that_never_arrives_times_out(ctx, backend):
    """Rank 0 of a world of two whose "peer" window is just a second local buffer: nobody ever
    raises rank 1's flag.  The wait must run out (limit lowered to ~0.1 ms for the test), the
    call must report DEVICE_LOST with status 0x7C050005, the tensor must be unchanged, and the
    context must keep working."""
    v = (np.arange(1024, dtype=np.float32) / 3).astype(np.float16)
    buf = ctx.upload(v)
    comm, _ = ctx.peer_comm_create(0, 2, v.nbytes)
    nbytes = int(backend.lib.lux_cuda_peer_comm_window_bytes(comm))
    fake = ctx.upload(np.zeros(nbytes, np.uint8))             # stands in for rank 1's window
    backend.tune("peer_wait_limit", 2000)
    try:
        ctx.peer_comm_connect_ptrs(comm, [ctx.peer_comm_window(comm), fake.device_ptr])
        with pytest.raises(B.BackendError) as e:
            ctx.peer_allreduce(comm, buf, v.size, B.F16)
        assert e.value.code == B.DEVICE_LOST
        assert ctx.last_device_status() == 0x7C050005
        assert np.array_equal(buf.to_host(np.float16, v.shape), v)
        # rank 0 did push: its slot in the stand-in window holds {4 bytes of the tensor, epoch 1} words
        win = fake.to_host(np.uint8, (nbytes,))
        slot_bytes = 2 * ((v.nbytes + 255) // 256 * 256)
        parity, src = 1, 0                                    # first epoch is 1
        off = (parity * 2 + src) * slot_bytes
        words = win[off:off + 2 * v.nbytes].view(np.uint32).reshape(-1, 2)
        assert np.array_equal(words[:, 0], v.view(np.uint32))
        assert (words[:, 1] == 1).all()
    finally:
        backend.tune("peer_wait_limit", 0)
        ctx.peer_comm_destroy(comm)
    # the context is still good for ordinary work
    x, layer = synth.activations(1, 512, "f16", 3, "after.x"), synth.int4_layer(64, 512, 3, "after")
    L, xb = ctx.upload_layer(layer), ctx.upload(x)
    yb = ctx.alloc(64 * 2)
    ctx.qmatmul(xb, L, yb, 1, B.F16, B.F16)
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    assert orc.rel_l2(yb.to_host(np.float16, (1, 64)), ref) < 5e-3
