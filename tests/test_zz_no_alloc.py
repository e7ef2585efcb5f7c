"""lux_cuda_qmlp_noalloc: the FFN entry point for callers that cannot allocate device memory
(hosts whose arena already owns all of it, decode loops that must not hit cudaMalloc's
device-wide synchronisation).  Its scratch is a fixed array inside the library, shared by
all calls, so the checks are: same answer as lux_cuda_qmlp with a caller-provided scratch,
on two calls in a row with different inputs (the array keeps the first call's contents),
and a clear refusal when the scratch would not fit.

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from webgpu_b200 import backend as B
from webgpu_b200 import synth

pytestmark = pytest.mark.gpu
TOL_16 = 5e-3


def _run_pair(ctx, G, D, x, K, I, H, M):
    xb = ctx.upload(x)
    hb = ctx.alloc(M * I * 2)
    y_ref_b, y_new_b = ctx.alloc(M * H * 2), ctx.alloc(M * H * 2)
    ctx.qmlp(xb, G, D, hb, y_ref_b, M, B.F16)
    ctx.qmlp_noalloc(xb, G, D, y_new_b, M, B.F16)
    return y_ref_b.to_host(np.float16, (M, H)), y_new_b.to_host(np.float16, (M, H))


@pytest.mark.parametrize("M", [1, 5])
def test_noalloc_matches_existing_entry_point_twice(ctx, M):
    K, I, H = 512, 768, 256
    gate_up, down = synth.mlp_layers(K, I, H, 41, "na")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    for call, seed in enumerate((41, 42)):            # second call: new x over the stale scratch
        x = synth.activations(M, K, "f16", seed, f"na.x{call}")
        y_ref, y_new = _run_pair(ctx, G, D, x, K, I, H, M)
        assert orc.rel_l2(y_new, y_ref) < TOL_16
        assert orc.rel_l2(y_new, orc.mlp(x, gate_up.triple, down.triple, fused=True)) < TOL_16


def test_noalloc_holds_device_memory_constant_at_tensor_core_batches(ctx, backend):
    """Batch 16 takes the tensor-core route (which also uses the context's split-K exchange
    buffer, allocated with the context): the call must leave the device's free memory exactly as
    it found it, and agree with the allocating entry point.  The first call on a device resolves
    the scratch array's address, so the measurement brackets a later call."""
    K, I, H, M = 1024, 2048, 512, 16
    gate_up, down = synth.mlp_layers(K, I, H, 44, "na.tc")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    x = synth.activations(M, K, "f16", 44, "na.tc.x")
    xb, hb = ctx.upload(x), ctx.alloc(M * I * 2)
    y_ref_b, y_new_b = ctx.alloc(M * H * 2), ctx.alloc(M * H * 2)
    ctx.qmlp(xb, G, D, hb, y_ref_b, M, B.F16)
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    ctx.qmlp_noalloc(xb, G, D, y_new_b, M, B.F16)              # first call: set-up
    free_before = ctx.device_info()["memory_available"]
    for _ in range(3):
        ctx.qmlp_noalloc(xb, G, D, y_new_b, M, B.F16)
    assert ctx.device_info()["memory_available"] == free_before
    assert backend.last_kernel_name() == "lux_qgemm_i4_tc_wa_f16"
    y_ref, y_new = y_ref_b.to_host(np.float16, (M, H)), y_new_b.to_host(np.float16, (M, H))
    assert np.array_equal(y_new.view(np.uint16), y_ref.view(np.uint16))
    assert orc.rel_l2(y_new, orc.mlp(x, gate_up.triple, down.triple, fused=True, w_round=orc.F16)) < TOL_16


def test_noalloc_rejects_oversized_scratch(ctx):
    K, H = 256, 128
    I = B.NOALLOC_MAX_BYTES // 2 // 4 + 128           # M * I * 2 just over the limit for M = 4
    gate_up, down = synth.mlp_layers(K, I, H, 43, "na.big")
    G, D = ctx.upload_layer(gate_up), ctx.upload_layer(down)
    xb = ctx.upload(synth.activations(4, K, "f16", 43, "na.big.x"))
    yb = ctx.alloc(4 * H * 2)
    with pytest.raises(B.BackendError) as e:
        ctx.qmlp_noalloc(xb, G, D, yb, 4, B.F16)
    assert e.value.code == B.INVALID_ARGUMENT
    ctx.qmlp_noalloc(xb, G, D, yb, 3, B.F16)          # 3 * I * 2 fits
