"""Multi-GPU layer: one process per GPU, torch.distributed (NCCL over NVLink) for the plumbing.

The reference is single-GPU (no NCCL/MPI anywhere; its device/default_fft.h:14 only has a
"support multi nodes" to-do), so this layer has no reference counterpart; it is built from
the single-GPU plan (the C ABI) plus three helper kernels.

* Batched transforms shard by batch: `shard_range` gives each rank a contiguous range of
  signals and the rank runs an ordinary Plan on it.  No communication.
* One transform too large for a GPU uses the four-step decomposition over N = N1 * N2 seen
  as an N1 x N2 row-major matrix whose rows are block-distributed:
    1. all-to-all so that each rank holds N2/P columns with all N1 rows, transposed locally
       to [N2/P][N1]
    2. N2/P local FFTs of length N1 (a Plan, FT on if asked), then a transpose fused with the
       twiddle W_N^(n2*k1) giving [N1][N2/P]
    3. all-to-all back: each rank holds N1/P values of k1 with all n2, [N1/P][N2]
    4. N1/P local FFTs of length N2
  The result is X[k1 + N1*k2] at rank(k1), position [k1_local][k2] ("transposed out", what
  FFTW-MPI and cuFFTMp call it); natural_order=True adds a third exchange that leaves each
  rank with its contiguous slab of X.
The all-to-all is torch.distributed.all_to_all_single; every kernel touches local memory
only (remote data always lands in local HBM first).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Tuple

from . import _lib
from ._lib import lib


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of `total` items for `rank`; sizes differ by at most one."""
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def split_log(logn: int) -> Tuple[int, int]:
    """(log2 N1, log2 N2) with N1 >= N2: 2^30 -> 2^15 x 2^15, 2^29 -> 2^15 x 2^14."""
    l1 = (logn + 1) // 2
    return l1, logn - l1


class DeviceBackend:
    """Local operations of the four-step transform on CUDA tensors, through the C ABI."""

    def __init__(self, dtype_code: int, device_index: int, if_ft: int = 0, if_err: int = 0, thread_bs: int = 1):
        import torch

        from . import Plan

        self.torch = torch
        self.Plan = Plan
        self.dt = dtype_code
        self.dev = device_index
        self.if_ft, self.if_err, self.thread_bs = if_ft, if_err, thread_bs
        self.plans = {}

    def _stream(self):
        return self.torch.cuda.current_stream(self.dev).cuda_stream

    def empty_like(self, x):
        return self.torch.empty_like(x)

    def fft_rows(self, x, logn: int):
        """FFT of every contiguous length-2^logn row of x (any leading shape)."""
        batch = x.numel() >> logn
        key = (logn, batch)
        if key not in self.plans:
            self.plans[key] = self.Plan(logn, batch, self.dt, self.if_ft, self.if_err, self.thread_bs, device=self.dev)
        out = self.torch.empty_like(x)
        self.plans[key].exec_ptr(x.data_ptr(), out.data_ptr(), self._stream())
        return out

    def transpose(self, x, rows: int, cols: int):
        out = self.torch.empty_like(x)
        _lib.check(lib().tfft_transpose(x.data_ptr(), out.data_ptr(), rows, cols, self.dt, self._stream()), "tfft_transpose")
        return out

    def twiddle_transpose(self, x, rows: int, cols: int, row0: int, col0: int, log_total: int):
        out = self.torch.empty_like(x)
        _lib.check(lib().tfft_twiddle_transpose(x.data_ptr(), out.data_ptr(), rows, cols, row0, col0, log_total, self.dt,
                                                self._stream()), "tfft_twiddle_transpose")
        return out

    def permute102(self, x, a: int, b: int, run: int):
        out = self.torch.empty_like(x)
        _lib.check(lib().tfft_permute102(x.data_ptr(), out.data_ptr(), a, b, run, self.dt, self._stream()), "tfft_permute102")
        return out

    def all_to_all(self, x, group):
        import torch.distributed as dist

        out = self.torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    def ft_counts(self):
        """(blocks that detected, tiles recomputed) summed over the local plans' last runs."""
        nd = nc = 0
        for p in self.plans.values():
            d, c, _ = p.ft_status()
            nd += d
            nc += c
        return nd, nc


class FourStepFFT:
    """Distributed 1-D FFT of length 2^logn over the ranks of `group`.

    Input: this rank's rows of the N1 x N2 matrix, i.e. elements
    [rank*N/P, (rank+1)*N/P) of the signal.  Output: see module docstring.
    `backend` supplies the local operations (DeviceBackend on GPUs; tests inject a host
    stand-in to check the distribution logic with gloo).
    """

    def __init__(self, logn: int, world: int, rank: int, backend, group=None, natural_order: bool = False):
        self.logn, self.world, self.rank = logn, world, rank
        self.l1, self.l2 = split_log(logn)
        self.n1, self.n2 = 1 << self.l1, 1 << self.l2
        if self.n1 % world or self.n2 % world:
            raise ValueError("world size must divide both factors of the transform")
        self.be, self.group, self.natural = backend, group, natural_order
        if world > 1:
            self._agree()

    def _agree(self):
        """Every rank must describe the same transform: a rank built with another length or output
        order would exchange blocks of the wrong shape (silently wrong data, or a collective that
        never completes).  One all_gather of the description at construction; any difference raises
        on every rank."""
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            return
        mine = (self.logn, self.world, bool(self.natural))
        seen = [None] * self.world
        dist.all_gather_object(seen, mine, group=self.group)
        if any(s != mine for s in seen):
            raise ValueError(f"ranks disagree on the transform (logn, world, natural_order): {seen}")

    def __call__(self, x_local):
        be, P, r = self.be, self.world, self.rank
        n1, n2, n1l, n2l = self.n1, self.n2, self.n1 // P, self.n2 // P
        # 1. [n1l][P][n2l] -> [P][n1l][n2l], exchange, recv = [N1][n2l], transpose -> [n2l][N1]
        a = be.permute102(x_local, n1l, P, n2l)
        a = self._exchange(a)
        a = be.transpose(a, n1, n2l)
        # 2. FFT over n1, then twiddle W_N^(n2*k1) fused with the transpose -> [N1][n2l]
        a = be.fft_rows(a, self.l1)
        a = be.twiddle_transpose(a, n2l, n1, r * n2l, 0, self.logn)
        # 3. rows k1 of rank j are contiguous: exchange, recv = [P][n1l][n2l] -> [n1l][P][n2l] = [n1l][N2]
        a = self._exchange(a)
        a = be.permute102(a, P, n1l, n2l)
        # 4. FFT over n2 -> Z[k1_local][k2]
        a = be.fft_rows(a, self.l2)
        if not self.natural:
            return a
        # natural order: X[k1 + N1*k2]; rank j gets k2 in its range: pack, exchange, transpose
        a = be.permute102(a, n1l, P, n2l)
        a = self._exchange(a)
        return be.transpose(a, n1, n2l)      # [k2_local][k1] = this rank's slab of X

    def _exchange(self, a):
        return a if self.world == 1 else self.be.all_to_all(a, self.group)

    def output_index(self, k1_local: int, k2: int) -> int:
        """Global frequency index of element [k1_local][k2] of the transposed-out result."""
        return (self.rank * (self.n1 // self.world) + k1_local) + self.n1 * k2


def dma_piece_geometry(rows: int, cols: int, ld: int, row0: int, world: int, pieces: int, g: int, j: int):
    """Element offsets and extents of the 2-D copy that carries piece g of one exchange to receiver j.

    The sender's [rows][cols] matrix is packed per receiver as [cols / world][rows]; receiver j's
    buffer holds [cols / world] lines of pitch ld and this sender's rows start at row0 in a line.
    Returns (dst_offset, dst_pitch, src_offset, src_pitch, width, height), offsets and pitches in
    elements: dst_offset into receiver j's buffer, src_offset into the sender's send buffer.
    """
    cb = cols // world
    piece = cb // pieces
    return (g * piece * ld + row0, ld, (j * cb + g * piece) * rows, rows, rows, piece)


class PeerBuffers:
    """Two receive buffers per rank that every other rank of the node can store into.

    Allocated with tfft_peer_alloc (plain cudaMalloc, so the CUDA IPC handle points at the
    start), handles exchanged with one all_gather, peers mapped with tfft_peer_open.
    """

    def __init__(self, nbytes: int, world: int, rank: int, device_index: int, group=None):
        import torch
        import torch.distributed as dist

        self.world, self.rank, self.nbytes = world, rank, nbytes
        self.local = []
        self.peers = []   # per buffer: list of `world` pointers
        self._opened = []
        for _ in range(2):
            p = C.c_void_p()
            _lib.check(lib().tfft_peer_alloc(nbytes, C.byref(p)), "tfft_peer_alloc")
            self.local.append(p.value)
        for b in range(2):
            ptrs = [None] * world
            ptrs[rank] = self.local[b]
            if world > 1:
                h = (C.c_ubyte * 64)()
                _lib.check(lib().tfft_peer_export(self.local[b], h), "tfft_peer_export")
                mine = torch.tensor(list(h), dtype=torch.uint8, device=f"cuda:{device_index}")
                allh = torch.empty(world * 64, dtype=torch.uint8, device=mine.device)
                dist.all_gather_into_tensor(allh, mine, group=group)
                allh = allh.cpu().numpy().reshape(world, 64)
                for j in range(world):
                    if j == rank:
                        continue
                    hb = (C.c_ubyte * 64)(*allh[j].tolist())
                    q = C.c_void_p()
                    _lib.check(lib().tfft_peer_open(hb, C.byref(q)), "tfft_peer_open")
                    ptrs[j] = q.value
                    self._opened.append(q.value)
            self.peers.append(ptrs)
        if world > 1:
            dist.barrier(group=group)

    def table(self, b: int):
        return (C.c_void_p * self.world)(*self.peers[b])

    def close(self):
        for q in self._opened:
            lib().tfft_peer_close(q)
        self._opened = []
        for p in self.local:
            lib().tfft_peer_free(p)
        self.local = []


class FusedFourStepFFT(FourStepFFT):
    """Four-step transform whose exchanges are fused into the transposing kernels.

    Each all-to-all of FourStepFFT, together with the pack before it and the transpose after
    it, becomes ONE kernel (tfft_scatter_transpose) that applies the twiddle, transposes
    through shared memory and stores every tile straight into the receiving GPU's buffer over
    NVLink; a one-element all_reduce behind it orders the receivers' next kernel after all
    senders.  Local HBM passes per transform drop from ten to six and the transfer overlaps
    the kernel that produces the data.  Same input and output conventions as FourStepFFT.
    """

    def __init__(self, logn: int, world: int, rank: int, dtype_code: int, device_index: int, group=None,
                 natural_order: bool = False, if_ft: int = 0, if_err: int = 0, thread_bs: int = 1, pipeline: int = 1,
                 exchange: str = "stores"):
        """pipeline = G > 1 cuts each exchange into G column groups issued on a side stream; the
        local transforms of group g run on the caller's stream while group g + 1 is in flight.

        exchange (pipelined form only): "stores" = the transposing kernel stores into the peers'
        buffers itself; "dma" = it packs into a local send buffer (own share straight into the own
        receive buffer) and the copy engines move each peer's block with one 2-D copy, which leaves
        the SMs to the transforms."""
        import torch

        be = DeviceBackend(dtype_code, device_index, if_ft, if_err, thread_bs)
        super().__init__(logn, world, rank, be, group, natural_order)
        if (self.n1 // world) % 32 or (self.n2 // world) % 32:
            raise ValueError("each rank's share of both factors must be a multiple of 32")
        self.torch, self.dt, self.dev = torch, dtype_code, device_index
        self.esize = 8 if dtype_code == 0 else 16
        self.bufs = PeerBuffers((self.n1 * self.n2 // world) * self.esize, world, rank, device_index, group)
        self.token = torch.zeros(1, device=f"cuda:{device_index}")
        self._plans = {}
        self.G = max(1, int(pipeline))
        if self.G > 1:
            if (self.n1 // world) % (32 * self.G) or (self.n2 // world) % (32 * self.G):
                raise ValueError("pipeline groups must hold a multiple of 32 lines")
            # the exchange pieces run at low priority, the transforms behind them at high priority:
            # otherwise the blocks of piece g + 1, already queued, keep the transform of piece g
            # off the SMs until they have drained and nothing overlaps
            self.side = torch.cuda.Stream(device=device_index, priority=0)
            self.fast = torch.cuda.Stream(device=device_index, priority=-1)
            # the exchange kernel is NVLink bound: a few resident blocks per SM saturate the links
            sms = torch.cuda.get_device_properties(device_index).multi_processor_count
            self.copy_blocks = int(os.environ.get("TFFT_EXCHANGE_BLOCKS_PER_SM", "4")) * sms
        if exchange not in ("stores", "dma"):
            raise ValueError("exchange must be 'stores' or 'dma'")
        self.exchange = exchange if self.G > 1 and world > 1 else "stores"
        if self.exchange == "dma":
            self.send = torch.empty((self.n1 * self.n2 // world) * self.esize, dtype=torch.uint8, device=f"cuda:{device_index}")
            self.copy = torch.cuda.Stream(device=device_index, priority=0)
            self.fence_stream = torch.cuda.Stream(device=device_index, priority=-1)
            # here the pack kernels feed the copy engines, so they go first and the transforms fill in
            self.side = torch.cuda.Stream(device=device_index, priority=-1)
            self.fast = torch.cuda.Stream(device=device_index, priority=0)

    def _stream(self):
        return self.torch.cuda.current_stream(self.dev).cuda_stream

    def _fence(self):
        # stream-ordered barrier: nobody's next kernel starts before everybody's stores are issued and complete
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(self.token, group=self.group)

    def _scatter(self, src_ptr, buf, rows, cols, ld, row0, tw, sub_off=None, sub_len=None, max_blocks=0):
        if sub_off is None:
            sub_off, sub_len = 0, cols // self.world
        _lib.check(lib().tfft_scatter_transpose_part(src_ptr, self.bufs.table(buf), self.world, rows, cols, ld, row0, int(tw),
                                                     self.logn, sub_off, sub_len, max_blocks, self.dt, self._stream()),
                   "tfft_scatter_transpose_part")

    def _plan(self, logn, count):
        from . import Plan

        key = (logn, count)
        if key not in self._plans:
            self._plans[key] = Plan(logn, count, self.dt, self.be.if_ft, self.be.if_err, self.be.thread_bs, device=self.dev)
            self._plans[key].set_ft_accumulate(True)
        return self._plans[key]

    def _exchange_and_transform(self, src, buf, rows, cols, ld, row0, tw, line_log, lines, out):
        """One pipelined exchange: G scatter pieces + fences on the side stream, and behind each
        fence the transform of the lines that piece completed, on the caller's stream."""
        torch, G = self.torch, self.G
        main = torch.cuda.current_stream(self.dev)
        self.side.wait_stream(main)
        piece = (cols // self.world) // G          # lines of the receiver completed by one piece
        events = []
        with torch.cuda.stream(self.side):
            for g in range(G):
                self._scatter(src.data_ptr(), buf, rows, cols, ld, row0, tw, g * piece, piece, self.copy_blocks)
                self._fence()
                ev = torch.cuda.Event()
                ev.record(self.side)
                events.append(ev)
        plan = self._plan(line_log, piece)
        step = piece * (1 << line_log) * self.esize
        self.fast.wait_stream(main)
        for g in range(G):
            self.fast.wait_event(events[g])
            plan.exec_ptr(self.bufs.local[buf] + g * step, out.data_ptr() + g * step, self.fast.cuda_stream)
        main.wait_stream(self.fast)
        return out

    def _exchange_dma(self, src, buf, rows, cols, ld, row0, tw, line_log, out):
        """The pipelined exchange with the copy engines as movers.  Piece g: (side stream) pack
        kernel -> (copy stream) one 2-D copy per peer, nearest rank first so that no two senders
        aim at one receiver at a time -> (fence stream) barrier -> (fast stream) transform."""
        torch, G, P, r, es = self.torch, self.G, self.world, self.rank, self.esize
        main = torch.cuda.current_stream(self.dev)
        for s in (self.side, self.copy, self.fence_stream, self.fast):
            s.wait_stream(main)
        cb = cols // P
        piece = cb // G
        # "receivers" of the pack kernel: the send buffer's block for peer j (pitch rows), the own
        # receive buffer for j == rank (pitch ld, offset row0)
        ptrs = (C.c_void_p * P)(*[self.bufs.local[buf] if j == r else self.send.data_ptr() + j * cb * rows * es
                                  for j in range(P)])
        lds = (C.c_longlong * P)(*[ld if j == r else rows for j in range(P)])
        offs = (C.c_longlong * P)(*[row0 if j == r else 0 for j in range(P)])
        events = []
        for g in range(G):
            with torch.cuda.stream(self.side):
                _lib.check(lib().tfft_scatter_transpose_ex(src.data_ptr(), ptrs, lds, offs, P, rows, cols, row0, int(tw),
                                                           self.logn, g * piece, piece, 0, self.dt, self.side.cuda_stream),
                           "tfft_scatter_transpose_ex")
                packed = torch.cuda.Event()
                packed.record(self.side)
            self.copy.wait_event(packed)
            for k in range(1, P):
                j = (r + k) % P
                doff, dpitch, soff, spitch, width, height = dma_piece_geometry(rows, cols, ld, row0, P, G, g, j)
                _lib.check(lib().tfft_copy_2d(self.bufs.peers[buf][j] + doff * es, dpitch * es, self.send.data_ptr() + soff * es,
                                              spitch * es, width * es, height, self.copy.cuda_stream), "tfft_copy_2d")
            sent = torch.cuda.Event()
            sent.record(self.copy)
            self.fence_stream.wait_event(sent)
            with torch.cuda.stream(self.fence_stream):
                self._fence()
                ev = torch.cuda.Event()
                ev.record(self.fence_stream)
            events.append(ev)
        plan = self._plan(line_log, piece)
        step = piece * (1 << line_log) * es
        for g in range(G):
            self.fast.wait_event(events[g])
            plan.exec_ptr(self.bufs.local[buf] + g * step, out.data_ptr() + g * step, self.fast.cuda_stream)
        main.wait_stream(self.fast)
        main.wait_stream(self.side)
        main.wait_stream(self.copy)
        main.wait_stream(self.fence_stream)
        return out

    def _fft_from(self, src_ptr, logn, count, out):
        self._plan(logn, count).exec_ptr(src_ptr, out.data_ptr(), self._stream())
        return out

    def __call__(self, x_local):
        P, r = self.world, self.rank
        n1, n2, n1l, n2l = self.n1, self.n2, self.n1 // P, self.n2 // P
        x_local = x_local.contiguous()
        if self.G > 1:
            if self.exchange == "dma":
                tmp = self._exchange_dma(x_local, 0, n1l, n2, n1, r * n1l, False, self.l1, self.torch.empty_like(x_local))
                out = self._exchange_dma(tmp, 1, n2l, n1, n2, r * n2l, True, self.l2, self.torch.empty_like(x_local))
            else:
                tmp = self._exchange_and_transform(x_local, 0, n1l, n2, n1, r * n1l, False, self.l1, n2l,
                                                   self.torch.empty_like(x_local))
                out = self._exchange_and_transform(tmp, 1, n2l, n1, n2, r * n2l, True, self.l2, n1l,
                                                   self.torch.empty_like(x_local))
            self.torch.cuda.current_stream(self.dev).wait_stream(self.side)
            if not self.natural:
                return out
            self._scatter(out.data_ptr(), 0, n1l, n2, n1, r * n1l, False)
            self._fence()
            res = self.torch.empty_like(x_local)
            _lib.check(lib().tfft_stream_copy(self.bufs.local[0], res.data_ptr(), res.numel() * self.esize, self._stream()),
                       "tfft_stream_copy")
            self._fence()   # see the end of this method
            return res
        # 1. x[n1l][N2] -> every rank's buffer 0 as [n2l][N1]
        self._scatter(x_local.data_ptr(), 0, n1l, n2, n1, r * n1l, False)
        self._fence()
        # 2. FFT over n1
        tmp = self._fft_from(self.bufs.local[0], self.l1, n2l, self.torch.empty_like(x_local))
        # 3. twiddle W_N^(n2*k1) + transpose -> every rank's buffer 1 as [n1l][N2]
        self._scatter(tmp.data_ptr(), 1, n2l, n1, n2, r * n2l, True)
        self._fence()
        # 4. FFT over n2 -> Z[k1_local][k2]
        out = self._fft_from(self.bufs.local[1], self.l2, n1l, tmp)
        if not self.natural:
            return out
        self._scatter(out.data_ptr(), 0, n1l, n2, n1, r * n1l, False)
        self._fence()
        res = self.torch.empty_like(x_local)
        # device-to-device copy of this rank's slab out of the receive buffer (stream ordered)
        _lib.check(lib().tfft_stream_copy(self.bufs.local[0], res.data_ptr(), res.numel() * self.esize, self._stream()),
                   "tfft_stream_copy")
        # The copy reads receive buffer 0, which the NEXT call's first exchange overwrites from
        # every peer.  Without a barrier here a faster peer's stores could land while this rank
        # still copies out (write after read across GPUs), so all ranks meet once more.
        self._fence()
        return res

    def ft_counts(self):
        """(detected, corrected) summed over every local transform since the last call of this
        method: the plans run once per pipeline piece and per pass, so they accumulate their
        counters (tfft_set_ft_accumulate) instead of keeping only the last run's."""
        nd = nc = 0
        for p in self._plans.values():
            d, c, _ = p.ft_status()
            nd += d
            nc += c
        return nd, nc

    def close(self):
        self.bufs.close()


class SingleProcessFourStep:
    """The same transform driven from ONE process over several devices (C ABI tfft_mg_*): rank r
    is position r of `devices`; a device may be listed more than once.  x_parts / results are
    lists of per-rank CUDA tensors of N / len(devices) elements."""

    def __init__(self, logn: int, dtype_code: int, devices, natural_order: bool = False, if_ft: int = 0, pipeline: int = 1):
        self.logn, self.dt, self.devices = logn, dtype_code, list(devices)
        self.l1, self.l2 = split_log(logn)
        self._h = C.c_void_p()
        arr = (C.c_int * len(self.devices))(*self.devices)
        _lib.check(lib().tfft_mg_plan_create(C.byref(self._h), logn, dtype_code, int(if_ft), len(self.devices), arr,
                                             int(natural_order), int(pipeline)), "tfft_mg_plan_create")

    def __call__(self, x_parts):
        import torch

        P = len(self.devices)
        outs = [torch.empty_like(x) for x in x_parts]
        for x in x_parts:                      # inputs were produced on torch's streams
            torch.cuda.synchronize(x.device)
        ins = (C.c_void_p * P)(*[x.data_ptr() for x in x_parts])
        ous = (C.c_void_p * P)(*[y.data_ptr() for y in outs])
        _lib.check(lib().tfft_mg_exec(self._h, ins, ous, None), "tfft_mg_exec")
        _lib.check(lib().tfft_mg_sync(self._h), "tfft_mg_sync")
        return outs

    def ft_counts(self):
        nd, nc = C.c_int(), C.c_int()
        _lib.check(lib().tfft_mg_ft_status(self._h, C.byref(nd), C.byref(nc)), "tfft_mg_ft_status")
        return nd.value, nc.value

    def close(self):
        if self._h:
            lib().tfft_mg_destroy(self._h)
            self._h = C.c_void_p()
