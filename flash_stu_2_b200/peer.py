"""Peer buffers of a tensor-parallel group for the token loop: the sub-layer outputs travel between the GPUs inside
the kernels that produce them (plain stores to peer memory over NVLink), not through a collective library.

Every rank owns one buffer (CUDA IPC makes it visible to the other ranks) holding, per exchange point of the token
step, an inbox `[world][rows][d]`, one arrival counter per sender, a send counter, a CTA counter and the exchange
descriptor its own producing kernels read.  Exchange points are used in a fixed order, once per token step, by every
rank; because a rank cannot send exchange e of the next step before it has received exchange e+1 (or the last one) of
this step from everybody, one inbox per exchange point is enough (at least two exchange points per step).

The reference is single-GPU; this replaces the all-gather / all-reduce a sharded copy of its sub-layers
(flash_stu/layers/stu_layer.py:78-98, flash_stu/layers/attention_layer.py) would need after each of them.
"""
import ctypes
import struct
from typing import List, Optional, Sequence

import torch

from . import _lib, ops

GATHER, REDUCE = "gather", "reduce"
MAX_PEERS = 8


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerExchange:
    """`kinds[e]` is GATHER (rank r contributes columns [r*d/world, (r+1)*d/world) of every row) or REDUCE (every
    rank contributes a full-width partial sum).  Build with `PeerExchange.connect` (one process per GPU) or
    `PeerExchange.emulate` (all ranks in one process on one GPU, for tests)."""

    def __init__(self, kinds: Sequence[str], rows: int, d: int, rank: int, world: int):
        if world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks")
        if len(kinds) < 2:
            raise ValueError("at least two exchange points per token step are needed for the inboxes to be safe")
        if d % (8 * world):
            raise ValueError("d must be a multiple of 8 * world")
        self.kinds, self.rows, self.d, self.rank, self.world = list(kinds), rows, d, rank, world
        E = len(kinds)
        self.desc_bytes = _lib.load().stu_peer_dest_bytes()
        assert self.desc_bytes == 8 + 16 * MAX_PEERS + 16
        self.off_inbox = 0
        self.off_flags = _align(E * world * rows * d * 2)
        self.off_epoch = self.off_flags + _align(E * world * 4)
        self.off_ctr = self.off_epoch + _align(E * 4)
        self.off_desc = self.off_ctr + _align(E * 4)
        # the single-launch exchange (push + wait + combine per row): counters per (exchange, sender, row), one epoch
        # per (exchange, row), one record per exchange
        self.xchg_bytes = _lib.load().stu_peer_xchg_bytes()
        assert self.xchg_bytes == 8 + 16 * MAX_PEERS + 8
        self.off_rflags = self.off_desc + _align(E * self.desc_bytes)
        self.off_repoch = self.off_rflags + _align(E * world * rows * 4)
        self.off_xdesc = self.off_repoch + _align(E * rows * 4)
        self.bytes = self.off_xdesc + _align(E * self.xchg_bytes)
        self.base: Optional[int] = None          # own buffer
        self.bases: List[int] = []               # every rank's buffer as mapped here
        self._opened: List[int] = []

    # ------------------------------------------------------------------ set-up
    def _allocate(self):
        p = ctypes.c_void_p()
        _lib.check(_lib.load().stu_peer_alloc(ctypes.byref(p), self.bytes), "stu_peer_alloc")
        self.base = p.value

    def _handle(self) -> bytes:
        h = ctypes.create_string_buffer(64)
        _lib.check(_lib.load().stu_peer_export(self.base, h), "stu_peer_export")
        return h.raw

    def _write_descriptors(self):
        E, w, r = len(self.kinds), self.world, self.rank
        blob = b""
        for e, kind in enumerate(self.kinds):
            slot, col = (0, r * (self.d // w)) if kind == GATHER else (r, 0)
            dest = [b + self.off_inbox + ((e * w + slot) * self.rows * self.d + col) * 2 for b in self.bases]
            flag = [b + self.off_flags + (e * w + r) * 4 for b in self.bases]
            pad = [0] * (MAX_PEERS - w)
            blob += struct.pack(f"ii{MAX_PEERS}Q{MAX_PEERS}QQQ", w, 0, *dest, *pad, *flag, *pad,
                                self.base + self.off_epoch + 4 * e, self.base + self.off_ctr + 4 * e)
        assert len(blob) == E * self.desc_bytes
        _lib.check(_lib.load().stu_peer_write(self.base + self.off_desc, blob, len(blob)), "stu_peer_write")
        blob = b""
        for e in range(E):
            inbox = [b + self.off_inbox + e * w * self.rows * self.d * 2 for b in self.bases]
            flag = [b + self.off_rflags + e * w * self.rows * 4 for b in self.bases]
            pad = [0] * (MAX_PEERS - w)
            blob += struct.pack(f"ii{MAX_PEERS}Q{MAX_PEERS}QQ", w, r, *inbox, *pad, *flag, *pad,
                                self.base + self.off_repoch + e * self.rows * 4)
        assert len(blob) == E * self.xchg_bytes
        _lib.check(_lib.load().stu_peer_write(self.base + self.off_xdesc, blob, len(blob)), "stu_peer_write")

    @classmethod
    def connect(cls, kinds, rows, d, group=None) -> "PeerExchange":
        """Collective over the process group (one process per GPU of one node): allocate, swap the inter-process
        handles, map the other ranks' buffers."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ex = cls(kinds, rows, d, rank, world)
        ex._allocate()
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, ex._handle(), group=group)
        for p, h in enumerate(handles):
            if p == rank:
                ex.bases.append(ex.base)
                continue
            q = ctypes.c_void_p()
            _lib.check(_lib.load().stu_peer_open(h, ctypes.byref(q)), "stu_peer_open")
            ex.bases.append(q.value)
            ex._opened.append(q.value)
        ex._write_descriptors()
        dist.barrier(group=group)   # nobody sends before every descriptor and zeroed counter is in place
        return ex

    @classmethod
    def emulate(cls, kinds, rows, d, world) -> List["PeerExchange"]:
        """All `world` ranks inside this process on the current GPU: for tests of the data path.  The producing
        kernels of every rank must be launched before any rank's combine (kernels that wait on one another cannot
        run as separate launches of one GPU)."""
        exs = [cls(kinds, rows, d, r, world) for r in range(world)]
        for ex in exs:
            ex._allocate()
        for ex in exs:
            ex.bases = [o.base for o in exs]
            ex._write_descriptors()
        return exs

    def close(self):
        lib = _lib.load()
        for q in self._opened:
            lib.stu_peer_close(q)
        self._opened = []
        if self.base is not None:
            lib.stu_peer_free(self.base)
            self.base = None

    # ------------------------------------------------------------------ use
    def dest(self, e: int) -> int:
        """Device address of the descriptor the producing kernel of exchange e takes."""
        return self.base + self.off_desc + e * self.desc_bytes

    def combine(self, e: int, x: torch.Tensor, norm_w: Optional[torch.Tensor] = None,
                xn: Optional[torch.Tensor] = None, eps: float = ops.RMS_EPS, wait_ms: int = 0):
        """x [rows, d] += what the ranks sent for exchange e; with norm_w also xn = RMSNorm(x) * norm_w."""
        w = self.world
        slots = 1 if self.kinds[e] == GATHER else w
        ops.peer_combine(x, self.base + self.off_inbox + e * w * self.rows * self.d * 2, self.rows * self.d, self.d,
                         slots, self.base + self.off_flags + e * w * 4, w, self.base + self.off_epoch + 4 * e,
                         norm_w, xn, eps, wait_ms)

    def exchange(self, e: int, x: torch.Tensor, src: torch.Tensor, norm_w: Optional[torch.Tensor] = None,
                 xn: Optional[torch.Tensor] = None, eps: float = ops.RMS_EPS, wait_ms: int = 0):
        """Exchange e in one launch: src [rows, d/world] (GATHER: this rank's channels) or [rows, d] (REDUCE: its
        partial sum) goes to every rank, x [rows, d] += everybody's rows, optionally xn = RMSNorm(x) * norm_w."""
        gather = self.kinds[e] == GATHER
        assert src.shape[1] == (self.d // self.world if gather else self.d)
        ops.peer_exchange(self.base + self.off_xdesc + e * self.xchg_bytes, x, src, gather, self.rows * self.d, norm_w,
                          xn, eps, wait_ms)

    def fake_arrival(self, e: int, sender: int, src: torch.Tensor, count: int):
        """Test aid: make it look as if rank `sender` had delivered `src` for exchange e, `count` times so far (host
        copies into this rank's inbox and counters).  Lets one GPU run a rank's exchange kernel without another
        kernel it would have to wait for."""
        w, rows, d = self.world, self.rows, self.d
        src = src.detach().to("cpu").contiguous()
        cols = src.shape[1]
        col, slot = (sender * cols, 0) if self.kinds[e] == GATHER else (0, sender)
        for row in range(rows):
            dst = self.base + self.off_inbox + (((e * w + slot) * rows + row) * d + col) * 2
            _lib.check(_lib.load().stu_peer_write(dst, src[row].view(torch.int16).numpy().tobytes(), cols * 2),
                       "stu_peer_write")
        blob = struct.pack(f"{rows}I", *([count] * rows))
        _lib.check(_lib.load().stu_peer_write(self.base + self.off_rflags + ((e * w + sender) * rows) * 4, blob,
                                              len(blob)), "stu_peer_write")

    def counters(self, e: int):
        """(arrival counters of exchange e, own send counter) read back from the device, for tests."""
        buf = ctypes.create_string_buffer(4 * self.world)
        _lib.check(_lib.load().stu_peer_read(buf, self.base + self.off_flags + e * self.world * 4, 4 * self.world),
                   "stu_peer_read")
        ep = ctypes.create_string_buffer(4)
        _lib.check(_lib.load().stu_peer_read(ep, self.base + self.off_epoch + 4 * e, 4), "stu_peer_read")
        return list(struct.unpack(f"{self.world}I", buf.raw)), struct.unpack("I", ep.raw)[0]
