"""Tensor-parallel Llama FFN over one process per GPU.

Sharding (Megatron-style, one exchange step):
  gate_up [2I, K]  column-parallel: rank r holds gate rows [r*I/t, (r+1)*I/t) AND the
                   matching up rows, stacked [gate_r ; up_r], so SwiGLU is local.
                   Quantization groups run along K and are untouched by the split.
  down    [H, I]   row-parallel: rank r holds input columns [r*I/t, (r+1)*I/t) of every
                   row, i.e. whole groups (I/t must be a multiple of the group size);
                   its output is a PARTIAL [M, H] sum.
  all-reduce(sum)  of the 16-bit partials finishes the layer: NCCL (NVLink/NVSwitch) through
                   torch.distributed, or the plugin's own one-shot push all-reduce over peer
                   memory (`collective="push"`, lux_cuda_peer_allreduce), which costs a few
                   microseconds instead of NCCL's ~11 for a 16 KB tensor.

The reference has no multi-device path at all (no NCCL/MPI call site anywhere in
luxcpp/webgpu); the `[gate ; up]` stacking is its own convention
(kernels/wgsl/steel/gemm/steel_gemm_fused.wgsl:525).  The compute runs through the
plugin's C ABI (lux_cuda_qmlp) on torch's current CUDA stream; torch owns the
activation buffers and `torch.distributed` does the collective.
"""
from __future__ import annotations

import numpy as np

from .synth import QLayer, pack_nibbles, unpack_nibbles


def shard_gate_up(layer: QLayer, rank: int, world: int) -> QLayer:
    """Rows [r*I/t, (r+1)*I/t) of gate and of up, stacked gate-then-up."""
    two_i = layer.N
    assert two_i % 2 == 0
    inter = two_i // 2
    assert inter % world == 0, "intermediate size must divide by the TP degree"
    loc = inter // world
    rows = np.r_[rank * loc:(rank + 1) * loc, inter + rank * loc:inter + (rank + 1) * loc]
    zeros = None if layer.zeros is None else np.ascontiguousarray(layer.zeros[rows])
    return QLayer(layer.bits, layer.group, 2 * loc, layer.K, np.ascontiguousarray(layer.w[rows]),
                  np.ascontiguousarray(layer.scales[rows]), zeros)


def shard_down(layer: QLayer, rank: int, world: int) -> QLayer:
    """Input columns [r*I/t, (r+1)*I/t) of every row; zero-points are re-packed because
    a shard may start at an odd group index."""
    K = layer.K
    assert K % world == 0
    kl = K // world
    assert kl % layer.group == 0, "a quantization group must not straddle two ranks"
    G = K // layer.group
    gl = kl // layer.group
    per_byte = 2 if layer.bits == 4 else 1
    w = np.ascontiguousarray(layer.w[:, rank * kl // per_byte:(rank + 1) * kl // per_byte])
    scales = np.ascontiguousarray(layer.scales[:, rank * gl:(rank + 1) * gl])
    zeros = None
    if layer.zeros is not None:
        zp = unpack_nibbles(layer.zeros, G)[:, rank * gl:(rank + 1) * gl]
        zeros = pack_nibbles(zp)
    return QLayer(layer.bits, layer.group, layer.N, kl, w, scales, zeros)


def shard_mlp(gate_up: QLayer, down: QLayer, rank: int, world: int):
    return shard_gate_up(gate_up, rank, world), shard_down(down, rank, world)


class PeerAllReduce:
    """The plugin's push all-reduce for one process per GPU on one node: creates this rank's
    window, exchanges the IPC handles through torch.distributed and connects.  ``__call__``
    sums a wrapped 16-bit buffer in place across the ranks on the plugin's current stream."""

    def __init__(self, ctx, rank: int, world: int, max_bytes: int, group=None):
        import torch.distributed as dist

        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self.comm, handle = ctx.peer_comm_create(rank, world, max_bytes)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle, group=group)
            ctx.peer_comm_connect(self.comm, b"".join(handles))
            dist.barrier(group=group)          # every window is mapped everywhere before the first push

    def __call__(self, buf, count: int, dtype: int, flags: int = 0) -> None:
        self.ctx.peer_allreduce(self.comm, buf, count, dtype, flags)

    def close(self) -> None:
        import torch
        import torch.distributed as dist

        if self.comm is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)  # nobody is still pushing into a window that goes away
            self.ctx.peer_comm_destroy(self.comm)
            self.comm = None


class TPMlp:
    """One rank's shard of the FFN, resident on this process's GPU.

    ``forward`` enqueues gate_up(+SwiGLU) and down on torch's current stream through the
    plugin and then all-reduces the partial output in place.  With ``world == 1`` no
    collective is issued.
    """

    def __init__(self, ctx, gate_up: QLayer, down: QLayer, rank: int, world: int, m_max: int,
                 act: str = "f16", group=None, presharded: bool = False, peer: "PeerAllReduce | None" = None):
        import torch
        from . import backend as B

        self.torch = torch
        self.B = B
        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self.peer = peer                     # None: torch.distributed (NCCL); else the push all-reduce
        self.act_code = {"f16": B.F16, "bf16": B.BF16}[act]
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16}[act]
        g_sh, d_sh = (gate_up, down) if presharded else shard_mlp(gate_up, down, rank, world)
        self.K, self.I, self.H = g_sh.K, g_sh.N // 2, d_sh.N
        self.gate_up = ctx.upload_layer(g_sh)
        self.down = ctx.upload_layer(d_sh)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.m_max = m_max
        self.x = torch.empty((m_max, self.K), dtype=tdt, device=dev)
        self.h = torch.empty((m_max, self.I), dtype=tdt, device=dev)
        self.y = torch.empty((m_max, self.H), dtype=tdt, device=dev)
        self._bx = ctx.wrap(self.x.data_ptr(), self.x.numel() * 2)
        self._bh = ctx.wrap(self.h.data_ptr(), self.h.numel() * 2)
        self._by = ctx.wrap(self.y.data_ptr(), self.y.numel() * 2)
        self.weight_bytes = self.gate_up.weight_bytes + self.down.weight_bytes

    def forward(self, M: int, all_reduce: bool = True):
        """x[:M] must already be in ``self.x``.  Returns the view ``self.y[:M]``."""
        torch = self.torch
        self.ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        out = self.y[:M]
        if all_reduce and self.world > 1 and self.peer is not None and (M * self.H) % 8 == 0:
            # FFN + push all-reduce in one call (the down kernel pushes from its epilogue at batch <= 2)
            self.ctx.qmlp_tp(self._bx, self.gate_up, self.down, self._bh, self._by, M, self.act_code,
                             self.peer.comm, flags=self.B.FLAG_NO_SYNC)
            return out
        self.ctx.qmlp(self._bx, self.gate_up, self.down, self._bh, self._by, M, self.act_code,
                      flags=self.B.FLAG_NO_SYNC)
        if all_reduce and self.world > 1:
            torch.distributed.all_reduce(out, group=self.group)
        return out


def all_ranks_agree(ok: bool, device=None, group=None) -> bool:
    """True only if `ok` holds on EVERY rank.  A choice that changes the sequence of collectives a
    rank issues (replay a captured graph or launch eagerly, use one collective or another) must be
    made with this, never per rank: ranks that issue different sequences wait for each other
    forever.  Call it on every rank, outside any try block."""
    import torch
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(ok)
    f = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(f, op=dist.ReduceOp.MIN, group=group)
    return int(f.item()) == 1


def all_reduce_partials(partial: np.ndarray, group=None) -> np.ndarray:
    """Host-side stand-in used by the CPU (gloo) tests of the sharding logic: sums f32
    partials across ranks with torch.distributed."""
    import torch
    import torch.distributed as dist

    t = torch.from_numpy(np.ascontiguousarray(partial, np.float32))
    dist.all_reduce(t, group=group)
    return t.numpy()
