"""Tensor-parallel FFN on two GPUs: one process per GPU, plugin kernels + NCCL all-reduce and,
second, the plugin's own push all-reduce over peer memory (repeatability, identical bits on
all ranks, CUDA-graph replay); rank 0 checks the results against the oracle's sharded
computation (tolerance 5e-3, f16)."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["REPO_ROOT"])
import numpy as np, torch
import torch.distributed as dist
from webgpu_b200 import backend as B, synth, tp

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
ctx = B.load().create_context(rank)
K, I, H = 1024, 2048, 512
gate_up, down = synth.mlp_layers(K, I, H, 51, "tp2")
for M in (1, 8, 64):
    x = synth.activations(M, K, "f16", 51, f"tp2.x{M}")
    mlp = tp.TPMlp(ctx, gate_up, down, rank, world, M, "f16")
    mlp.x[:M].copy_(torch.from_numpy(x).cuda())
    y = mlp.forward(M).float().cpu().numpy()
    torch.cuda.synchronize()
    if rank == 0:
        from oracle import oracle as orc
        shards = [tuple(l.triple for l in tp.shard_mlp(gate_up, down, r, world)) for r in range(world)]
        ref = orc.tp_mlp(x, shards, fused=True, w_round=orc.F16 if M > 32 else orc.F32)
        err = orc.rel_l2(y.astype(np.float16), ref)
        assert err < 5e-3, (M, err)
        print("TP_OK", M, err)
# ---- the plugin's own push all-reduce over peer memory instead of NCCL ----------------------
peer = tp.PeerAllReduce(ctx, rank, world, 64 * H * 2)
for M in (1, 8, 64):
    x = synth.activations(M, K, "f16", 51, f"tp2.x{M}")
    mlp = tp.TPMlp(ctx, gate_up, down, rank, world, M, "f16", peer=peer)
    mlp.x[:M].copy_(torch.from_numpy(x).cuda())
    outs = []
    for rep in range(5):                                   # several epochs: both parities, slot reuse
        outs.append(mlp.forward(M).float().cpu().numpy().copy())
        ctx.sync()                                         # raises DEVICE_LOST if a peer wait gave up
    assert all(np.array_equal(outs[0], o) for o in outs[1:]), "push all-reduce is not repeatable"
    assert ctx.last_device_status() == 0
    # every rank holds the same bits
    gathered = [None] * world
    dist.all_gather_object(gathered, outs[0].tobytes())
    assert all(g == gathered[0] for g in gathered), "ranks disagree"
    # captured in a CUDA graph and replayed (the epoch lives in device memory)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        mlp.forward(M)
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st, capture_error_mode="relaxed"):
            mlp.forward(M)
            mlp.forward(M)
        for _ in range(3):
            g.replay()
        st.synchronize()
        ctx.sync()
    assert np.array_equal(mlp.y[:M].float().cpu().numpy(), outs[0]), "graph replay differs"
    if rank == 0:
        from oracle import oracle as orc
        shards = [tuple(l.triple for l in tp.shard_mlp(gate_up, down, r, world)) for r in range(world)]
        ref = orc.tp_mlp(x, shards, fused=True, w_round=orc.F16 if M > 32 else orc.F32)
        err = orc.rel_l2(outs[0].astype(np.float16), ref)
        assert err < 5e-3, (M, err)
        print("PUSH_OK", M, err)
# ---- bf16 activations: up to four rows on the fixed-point GEMV, more on the tensor-core GEMM; the push
# all-reduce sums bf16 partial outputs ------------------------------------------------------------
for M in (1, 8):
    x = synth.activations(M, K, "bf16", 51, f"tp2.xb{M}")
    mlp = tp.TPMlp(ctx, gate_up, down, rank, world, M, "bf16", peer=peer)
    mlp.x[:M].copy_(torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16))
    y = mlp.forward(M).float().cpu().numpy().copy()
    ctx.sync()
    assert ctx.last_device_status() == 0
    gathered = [None] * world
    dist.all_gather_object(gathered, y.tobytes())
    assert all(g == gathered[0] for g in gathered), "ranks disagree (bf16)"
    if rank == 0:
        from oracle import oracle as orc
        shards = [tuple(l.triple for l in tp.shard_mlp(gate_up, down, r, world)) for r in range(world)]
        ref = synth.bf16_bits_to_f32(orc.tp_mlp(x, shards, fused=True, w_round=orc.F32 if M <= 4 else orc.BF16))
        err = orc.rel_l2(y, ref)
        assert err < 5e-3, (M, err)
        print("BF16_OK", M, err)
peer.close()
dist.barrier()
dist.destroy_process_group()
"""


def test_tp_two_gpus(tmp_path, backend):
    if backend.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, REPO_ROOT=ROOT, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert outs[0].count("TP_OK") == 3, outs[0]
    assert outs[0].count("PUSH_OK") == 3, outs[0]
    assert outs[0].count("BF16_OK") == 2, outs[0]
