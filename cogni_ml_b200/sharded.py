"""Row / vocabulary sharding of the quantized matmul over the GPUs of one box.

Output rows are independent (y[o] reads only row o of W and all of x), and rows are stored back to
back in the GGUF tensor, so rank g of G owns the contiguous row range shard_rows(N, g, G) — a
contiguous byte range of the raw tensor — and x is replicated.  There is exactly one exchange
step per matmul:

  * ShardedQuantWeight.gemv: each rank writes its [batch, rows] result into slot `rank` of a
    [G, batch, rows] buffer, one all-gather fills the other slots (NCCL over NVLink on GPUs);
  * ShardedLmHead.top1: each rank's fused GEMV + top-1 yields one int64 key per batch row,
    key = (orderable(value) << 32) | (0xFFFFFFFF - global_index); a MAX all-reduce of the keys
    picks the highest value and, among equal values, the lowest index — the reference's tie rule
    (src/ml/gguf/qwen35_cpu.cr:2052-2055).

One process per GPU, torch.distributed for the plumbing.  The local compute is a
DeviceQuantWeight; `local_factory` lets the host logic run under gloo on CPU in tests with a
stand-in for the device kernels.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .quant_matmul import QuantWeight, row_bytes


def shard_rows(out_dim: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous row range of `rank`: sizes differ by at most one row, earlier ranks get the extra."""
    if not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(out_dim, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_bytes(qw: QuantWeight, rank: int, world: int) -> np.ndarray:
    """The raw GGUF bytes of this rank's rows: a slice, never a repack."""
    r0, r1 = shard_rows(qw.out_dim, rank, world)
    rb = row_bytes(qw.type, qw.in_dim)
    return qw.raw[r0 * rb:r1 * rb]


def pack_top1_key(value: np.ndarray, index: np.ndarray) -> np.ndarray:
    """Host restatement of the device key: int64 (orderable(value) << 32) | (0xFFFFFFFF - index)."""
    value = np.asarray(value, dtype=np.float32) + np.float32(0.0)   # -0.0 -> +0.0
    bits = value.view(np.int32).astype(np.int64)
    ordv = np.where(bits >= 0, bits, bits ^ 0x7FFFFFFF)          # signed order == float order
    low = (0xFFFFFFFF - np.asarray(index, dtype=np.int64)) & 0xFFFFFFFF
    return (ordv << 32) | low


def unpack_top1_key(key: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    key = np.asarray(key, dtype=np.int64)
    ordv = (key >> 32).astype(np.int32)
    bits = np.where(ordv >= 0, ordv, ordv ^ 0x7FFFFFFF).astype(np.int32)
    index = (0xFFFFFFFF - (key & 0xFFFFFFFF)).astype(np.int64)
    return index.astype(np.int32), bits.view(np.float32)


def _default_factory(qw: QuantWeight, r0: int, r1: int, device):
    from .quant_matmul import DeviceQuantWeight
    return DeviceQuantWeight.upload(qw, device, r0, r1)


class ShardedQuantWeight:
    """This rank's row shard of a quantized weight plus the all-gather of the outputs."""

    def __init__(self, qw: QuantWeight, device, group: Optional[dist.ProcessGroup] = None,
                 local_factory: Callable = _default_factory):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out_dim, self.in_dim = qw.out_dim, qw.in_dim
        if qw.out_dim % self.world:
            raise ValueError("out_dim must divide evenly over the ranks for the gathered layout")
        self.rows = qw.out_dim // self.world
        self.r0, self.r1 = shard_rows(qw.out_dim, self.rank, self.world)
        self.device = torch.device(device)
        self.local = local_factory(qw, self.r0, self.r1, self.device)
        self._gather: Optional[torch.Tensor] = None

    def gather_buffer(self, batch: int) -> torch.Tensor:
        if self._gather is None or self._gather.shape[1] != batch:
            self._gather = torch.empty(self.world, batch, self.rows, dtype=torch.float32,
                                       device=self.device)
        return self._gather

    def gemv(self, x: torch.Tensor) -> torch.Tensor:
        """x f32 [batch, in_dim] (replicated) -> y f32 [batch, out_dim] on every rank."""
        batch = x.numel() // self.in_dim
        buf = self.gather_buffer(batch)
        self.local.gemv(x, out=buf[self.rank])
        if self.world > 1:
            dist.all_gather_into_tensor(buf.view(-1), buf[self.rank].reshape(-1), group=self.group)
        # [G, batch, rows] -> [batch, G*rows]: rank g's rows are columns [g*rows, (g+1)*rows)
        return buf.permute(1, 0, 2).reshape(batch, self.out_dim)


class ShardedLmHead:
    """Vocabulary-sharded fused lm_head: per-shard top-1, one MAX all-reduce of int64 keys."""

    def __init__(self, qw: QuantWeight, device, group: Optional[dist.ProcessGroup] = None,
                 local_factory: Callable = _default_factory):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.r0, self.r1 = shard_rows(qw.out_dim, self.rank, self.world)
        self.device = torch.device(device)
        self.in_dim = qw.in_dim
        self.local = local_factory(qw, self.r0, self.r1, self.device)

    def top2(self, x: torch.Tensor):
        """(index int32 [batch, 2], value f32 [batch, 2]) of the global best and runner-up: every
        shard contributes its two best keys, one all-gather, the two largest keys win."""
        _idx, _val, key = self.local.gemv_top2(x, want_keys=True)          # [batch, 2]
        if self.world > 1:
            allk = torch.empty(self.world, *key.shape, dtype=key.dtype, device=key.device)
            dist.all_gather_into_tensor(allk.view(-1), key.reshape(-1), group=self.group)
            key = allk.permute(1, 0, 2).reshape(key.shape[0], -1).topk(2, dim=1).values.contiguous()
        if key.is_cuda:
            from .quant_matmul import unpack_top1_keys
            idx, val = unpack_top1_keys(key.view(-1))
            return idx.view(-1, 2), val.view(-1, 2)
        idx, val = unpack_top1_key(key.numpy())
        return torch.from_numpy(idx.copy()), torch.from_numpy(val.copy())

    def top1(self, x: torch.Tensor):
        """(index int32 [batch], value f32 [batch]) of the global maximum, identical on all ranks."""
        _idx, _val, key = self.local.gemv_top1(x, want_keys=True)
        if self.world > 1:
            dist.all_reduce(key, op=dist.ReduceOp.MAX, group=self.group)
        if key.is_cuda:
            from .quant_matmul import unpack_top1_keys
            return unpack_top1_keys(key)
        idx, val = unpack_top1_key(key.numpy())
        return torch.from_numpy(idx.copy()), torch.from_numpy(val.copy())


# ----------------------------------------------------------------------------------------------
# The exchange fused into the GEMV launch (cogni_qmm_gemv_many_exchange): peer-mapped buffers.

def _make_exchange_struct():
    import ctypes as C

    class Exchange(C.Structure):   # struct cogni_qmm_exchange (include/cogni_qmm.h)
        _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("peer_offset", C.c_int64 * 8),
                    ("epoch", C.c_void_p), ("ticket", C.c_void_p)]
    return Exchange


_ExchangeStruct = _make_exchange_struct()


class PeerExchange:
    """One arena per rank, laid out identically on every rank and mapped into every process of the
    box (torch symmetric memory: the same physical allocation of rank g appears at buffer_ptrs[g] in
    every process, accessible from the local GPU): 256 bytes of state (this rank's epoch and
    ticket) followed by the gather buffers.  `buffer(name, batch, n)` hands out the same region on
    every rank, so an address offset inside the local arena is the offset inside every peer's.

    A gather buffer holds [batch][n] words of 8 bytes, (f32 value, u32 epoch): an exchanging launch
    writes each output as one such word on every GPU, and its consumer polls the words it reads for
    the epoch it expects (no fence, flag or barrier in between)."""

    STATE_BYTES = 256

    def __init__(self, nbytes: int, device, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("at most 8 ranks (the GPUs of one box)")
        self.device = torch.device(device)
        total = self.STATE_BYTES + ((nbytes + 255) // 256) * 256
        self._cursor = self.STATE_BYTES
        self._named = {}
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.arena = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self.arena.zero_()
            torch.cuda.synchronize(self.device)
            self._handle = symm_mem.rendezvous(self.arena, group if group is not None else dist.group.WORLD)
            ptrs = [int(v) for v in self._handle.buffer_ptrs]
            if ptrs[self.rank] != self.arena.data_ptr():
                raise RuntimeError("symmetric memory: the local buffer is not where the handle says")
            # every peer's arena through a torch view first: the same access path the kernels use
            for g in range(self.world):
                view = self._handle.get_buffer(g, (self.STATE_BYTES,), torch.uint8, 0)
                if int(view[128:192].sum().item()) != 0:
                    raise RuntimeError("symmetric memory: a peer's arena is not readable from here")
            self._handle.barrier()
        else:
            self.arena = torch.zeros(total, dtype=torch.uint8, device=self.device)
            torch.cuda.synchronize(self.device)
            ptrs = [self.arena.data_ptr()]
        ex = _ExchangeStruct()
        ex.world, ex.rank = self.world, self.rank
        base = ptrs[self.rank]
        for g in range(self.world):
            ex.peer_offset[g] = ptrs[g] - base
        ex.epoch = base + 64
        ex.ticket = base + 68
        self.struct = ex

    def buffer(self, name: str, batch: int, n: int) -> torch.Tensor:
        """The gather buffer `name` of the local arena as f32 [batch, n, 2]: [..., 0] the values,
        [..., 1] the epoch bits (allocated on first use; every rank must ask for the same names,
        shapes and order)."""
        if name not in self._named:
            nbytes = (batch * n * 8 + 255) // 256 * 256
            if self._cursor + nbytes > self.arena.numel():
                raise ValueError("exchange arena too small")
            self._named[name] = (self._cursor, batch, n)
            self._cursor += nbytes
        off, b, nn = self._named[name]
        return self.arena[off:off + b * nn * 8].view(torch.float32).view(b, nn, 2)

    def epoch(self) -> int:
        return int(self.arena[64:68].view(torch.int32).item())

    def unpack(self, buf: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """f32 [batch, n] values of a gather buffer written by the exchanging launch issued last on
        this exchange, on the stream's order (the unpacking kernel waits for the words itself)."""
        from ._lib import check, lib
        from .quant_matmul import _stream_ptr
        b, n, _ = buf.shape
        if out is None:
            out = torch.empty(b, n, dtype=torch.float32, device=buf.device)
        # the epoch of the exchange before this point of the stream is only known on the device;
        # read it in stream order
        epoch = torch.empty(1, dtype=torch.int32, device=buf.device)
        epoch.copy_(self.arena[64:68].view(torch.int32))
        check(lib.cogni_qmm_exchange_unpack(buf.data_ptr(), b * n, int(epoch.item()) & 0xFFFFFFFF,
                                            out.data_ptr(), _stream_ptr(stream)), "cogni_qmm_exchange_unpack")
        return out


class ExchangingGemv:
    """A prepared row-sharded qmatvec_many whose outputs reach every GPU inside the launch.

    weights: this rank's row shards (DeviceQuantWeight) of matrices that share x; outs: for each, a
    gather buffer (PeerExchange.buffer(name, batch, world * rows)): the launch writes this rank's
    columns [rank * rows, (rank + 1) * rows) of every batch row, locally and on every peer.
    x: plain f32 [batch, in_dim], or -- wait_previous -- the gather buffer [batch, in_dim, 2] that
    the exchanging launch issued just before this one wrote."""

    def __init__(self, exchange: PeerExchange, weights, x: torch.Tensor, outs, wait_previous: bool):
        import ctypes as C
        self.ex, self.weights, self.x, self.outs = exchange, list(weights), x, list(outs)
        w0 = self.weights[0]
        if len({(w.type, w.in_dim) for w in self.weights}) != 1:
            raise ValueError("weights must share type and in_dim")
        if len({w.out_dim for w in self.weights}) != 1:
            raise ValueError("the exchanged matrices of one launch must have equal row counts")
        self.batch = x.numel() // (w0.in_dim * (2 if wait_previous else 1))
        n = len(self.weights)
        total = exchange.world * w0.out_dim
        for o in self.outs:
            if tuple(o.shape) != (self.batch, total, 2) or not o.is_contiguous():
                raise ValueError("each output must be a gather buffer [batch, world * rows, 2]")
        self._w = (C.c_void_p * n)(*[w.raw.data_ptr() for w in self.weights])
        self._y = (C.c_void_p * n)(*[o[0, exchange.rank * w0.out_dim].data_ptr() for o in self.outs])
        self._n = (C.c_int * n)(*[w.out_dim for w in self.weights])
        self._pitch = total
        self._resident = int(all(w.resident for w in self.weights))
        self._wait = int(bool(wait_previous))

    def run(self, stream=None):
        import ctypes as C

        from ._lib import check, lib
        from .quant_matmul import _stream_ptr
        w0 = self.weights[0]
        check(lib.cogni_qmm_gemv_many_exchange(w0.type, len(self.weights), self._w, self.x.data_ptr(),
                                               None, 0, self._y, self._pitch, self._n, w0.in_dim,
                                               self.batch, self._resident, C.byref(self.ex.struct),
                                               self._wait, _stream_ptr(stream)),
              "cogni_qmm_gemv_many_exchange")
        return self.outs
