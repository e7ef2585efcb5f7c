"""World-size-2 run of the tensor-parallel sharding + all-reduce logic on CPU (gloo).

Each rank shards the FFN with webgpu_b200.tp, computes its partial with the oracle (the
stand-in for the GPU kernels, allowed only in tests) and all-reduces; rank 0 compares
with the unsharded oracle."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["REPO_ROOT"])
import numpy as np
import torch.distributed as dist
from oracle import oracle as orc
from webgpu_b200 import synth, tp

dist.init_process_group("gloo", init_method="env://")
rank, world = dist.get_rank(), dist.get_world_size()
K, I, H, M = 256, 512, 128, 3
gate_up, down = synth.mlp_layers(K, I, H, 11, "gloo")
x = synth.activations(M, K, "f16", 11, "gloo.x")
g_sh, d_sh = tp.shard_mlp(gate_up, down, rank, world)
partial = orc.mlp(x, g_sh.triple, d_sh.triple, fused=True)          # f16 partial, as a GPU would hand over
total = tp.all_reduce_partials(orc.to_f32(partial))
if rank == 0:
    ref = orc.mlp(x, gate_up.triple, down.triple, fused=True)
    err = orc.rel_l2(total.astype(np.float16), ref)
    assert err < 5e-3, err
    print("TP_GLOO_OK", err)
dist.barrier()
dist.destroy_process_group()
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tp_world2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, REPO_ROOT=ROOT, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "TP_GLOO_OK" in outs[0]


ORDER_WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["REPO_ROOT"])
import numpy as np
import torch.distributed as dist
from oracle import oracle as orc
from webgpu_b200 import synth, tp

dist.init_process_group("gloo", init_method="env://")
rank, world = dist.get_rank(), dist.get_world_size()
K, I, H, M = 256, 512, 128, 2
gate_up, down = synth.mlp_layers(K, I, H, 12, "order")
x = synth.activations(M, K, "f16", 12, "order.x")
g_sh, d_sh = tp.shard_mlp(gate_up, down, rank, world)
calls = []

def step():
    # one tensor-parallel FFN step: local kernels (the oracle stands in) + the all-reduce
    part = orc.to_f32(orc.mlp(x, g_sh.triple, d_sh.triple, fused=True))
    calls.append("all_reduce")
    return tp.all_reduce_partials(part)

def timed_region(capture_ok, steps):
    # the order of a benchmark's timed region: try to capture, AGREE, then replay or launch eagerly;
    # barriers outside the try.  Rank 1's capture "fails"; both ranks must then launch eagerly.
    dist.barrier(); calls.append("barrier")
    try:
        if not capture_ok:
            raise RuntimeError("capture refused")
        captured = True
    except RuntimeError:
        captured = False
    use_graph = tp.all_ranks_agree(captured)
    calls.append("graph" if use_graph else "eager")
    out = None
    for _ in range(steps):
        out = step()
    dist.barrier(); calls.append("barrier")
    return out

y1 = timed_region(capture_ok=(rank != 1), steps=3)      # one rank fails: everybody eager
y2 = timed_region(capture_ok=True, steps=2)             # nobody fails: everybody replays
assert calls.count("eager") == 1 and calls.count("graph") == 1, calls
seqs = [None] * world
dist.all_gather_object(seqs, calls)
assert all(s == seqs[0] for s in seqs), seqs              # every rank issued the same sequence
if rank == 0:
    ref = orc.mlp(x, gate_up.triple, down.triple, fused=True)
    assert orc.rel_l2(y1.astype(np.float16), ref) < 5e-3 and orc.rel_l2(y2.astype(np.float16), ref) < 5e-3
    print("TP_ORDER_OK")
dist.barrier()
dist.destroy_process_group()
"""


def test_capture_or_eager_is_decided_by_all_ranks(tmp_path):
    """The step order of the tensor-parallel benchmark over gloo, the oracle standing in for the
    kernels: when one rank's graph capture fails, every rank must fall back together, so that all
    ranks issue the same sequence of collectives and barriers and the run terminates."""
    script = tmp_path / "order_worker.py"
    script.write_text(ORDER_WORKER)
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, REPO_ROOT=ROOT, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "TP_ORDER_OK" in outs[0]
