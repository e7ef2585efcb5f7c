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
