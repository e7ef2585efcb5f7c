"""The plugin's push all-reduce on one GPU: the single-rank case, argument checking, the bounded
wait (a peer that never signals must end in a status word and DEVICE_LOST, with the tensor
untouched, the communicator marked failed and the context still usable), and the two-rank
arithmetic with the second rank played by the HOST: its words are written into rank 0's window
before the kernel runs, so no kernel ever waits for another kernel on the same GPU.  The real
two-process path runs in test_gpu_tp.py on two GPUs."""
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
    writes rank 1's words.  The wait must run out (deadline lowered to 2 ms for the test), the
    call must report DEVICE_LOST with status 0x7C050005, the tensor must be unchanged, a second
    call on the failed communicator must come back at once with the same answer, and the context
    must keep working."""
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
        # the failure is sticky: no second wait, the same report
        import time
        t0 = time.perf_counter()
        backend.tune("peer_wait_limit", 0)                    # back to the default of one second
        with pytest.raises(B.BackendError) as e2:
            ctx.peer_allreduce(comm, buf, v.size, B.F16)
        assert e2.value.code == B.DEVICE_LOST and time.perf_counter() - t0 < 0.5
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


def _slot_offset(world, max_bytes, parity, src):
    return (parity * world + src) * 2 * ((max_bytes + 255) // 256 * 256)


def _host_pushes(ctx, window_ptr, world, max_bytes, epoch, src, payload_f16):
    """What rank `src`'s kernel would store into a window for `epoch`: {4 bytes of payload, epoch} words."""
    words = np.empty((payload_f16.size // 2, 2), np.uint32)
    words[:, 0] = np.ascontiguousarray(payload_f16).view(np.uint32).ravel()
    words[:, 1] = epoch
    off = _slot_offset(world, max_bytes, epoch & 1, src)
    ctx.wrap(window_ptr + off, words.nbytes).from_host(words)


@pytest.mark.parametrize("count", [1024, 65536, 300 * 8])
def test_two_ranks_with_the_peer_played_by_the_host(ctx, backend, count):
    """World of two on one GPU: before each call the host writes rank 1's words for that epoch
    into rank 0's window, so the kernel finds them and never waits for another kernel.  Three
    epochs (both parities, slot reuse); 65536 elements take 32 CTAs, so the epoch is advanced by
    the last of several CTAs.  Result = f16(f32(a) + f32(b)) exactly."""
    rng = np.random.default_rng(7)
    nbytes = count * 2
    comm, _ = ctx.peer_comm_create(0, 2, nbytes)
    fake = ctx.upload(np.zeros(int(backend.lib.lux_cuda_peer_comm_window_bytes(comm)), np.uint8))
    try:
        win = ctx.peer_comm_window(comm)
        ctx.peer_comm_connect_ptrs(comm, [win, fake.device_ptr])
        for epoch in (1, 2, 3):
            a = rng.standard_normal(count).astype(np.float16)
            b = rng.standard_normal(count).astype(np.float16)
            _host_pushes(ctx, win, 2, nbytes, epoch, 1, b)
            buf = ctx.upload(a)
            ctx.peer_allreduce(comm, buf, count, B.F16)
            want = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
            assert np.array_equal(buf.to_host(np.float16, a.shape).view(np.uint16), want.view(np.uint16)), epoch
    finally:
        ctx.peer_comm_destroy(comm)


@pytest.mark.parametrize("mode,launches", [(0, 3), (1, 2)])
@pytest.mark.parametrize("M", [1, 2])
def test_fused_down_plus_allreduce_with_the_peer_played_by_the_host(ctx, backend, M, mode, launches):
    """lux_cuda_qmlp_tp at batch 1 and 2.  Default (mode 0): the down projection's kernel pushes its
    outputs from its epilogue and a reduce-only kernel waits and sums (three launches per FFN).
    Mode 1: the down kernel also waits for the peer's words and writes the sum (two launches).
    Rank 1's partial output is written into rank 0's window by the host beforehand; the result
    must be f16(f32(f16 partial of rank 0) + f32(partial of rank 1)) within the 16-bit tolerance
    of the oracle, on two calls in a row (two epochs)."""
    K, I, H = 1024, 2048, 512
    gate_up, down = synth.mlp_layers(K, I, H, 61, "fused")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    nbytes = M * H * 2
    comm, _ = ctx.peer_comm_create(0, 2, nbytes)
    fake = ctx.upload(np.zeros(int(backend.lib.lux_cuda_peer_comm_window_bytes(comm)), np.uint8))
    rng = np.random.default_rng(61)
    backend.tune("tp_fused_push", mode)
    try:
        win = ctx.peer_comm_window(comm)
        ctx.peer_comm_connect_ptrs(comm, [win, fake.device_ptr])
        for epoch in (1, 2):
            x = synth.activations(M, K, "f16", 61 + epoch, f"fused.x{epoch}")
            other = (rng.standard_normal((M, H)) * 0.05).astype(np.float16)
            _host_pushes(ctx, win, 2, nbytes, epoch, 1, other)
            xb, hb, yb = ctx.upload(x), ctx.alloc(M * I * 2), ctx.alloc(M * H * 2)
            before = backend.launch_count()
            ctx.qmlp_tp(xb, G, D, hb, yb, M, B.F16, comm)
            assert backend.launch_count() - before == launches, "the push was not fused into the down kernel"
            assert backend.last_kernel_name() == ("lux_qgemv_i4_g128_units_fx" if mode == 1 else "lux_peer_allreduce_push")
            y = yb.to_host(np.float16, (M, H))
            part = orc.mlp(x, gate_up.triple, down.triple, fused=True)
            want = (part.astype(np.float32) + other.astype(np.float32)).astype(np.float16)
            assert orc.rel_l2(y, want) < 5e-3, epoch
    finally:
        backend.tune("tp_fused_push", 0)
        ctx.peer_comm_destroy(comm)
