"""Multi-GPU layer: distribution logic on CPU ranks (gloo), kernels on one GPU, and a
2-GPU run where the machine has two."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
from oracle import fft_oracle as orc  # noqa: E402
from turbofft_b200 import multi_gpu as mg  # noqa: E402


def test_shard_range_covers_everything():
    for total, world in [(16, 4), (17, 4), (3, 8), (1 << 20, 8)]:
        spans = [mg.shard_range(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
    assert mg.split_log(30) == (15, 15) and mg.split_log(29) == (15, 14)


class HostBackend:
    """CPU stand-in for the device operations (numpy + the oracle FFT), used only to check
    the index logic and the all-to-all plumbing of FourStepFFT between gloo ranks."""

    def __init__(self, torch):
        self.torch = torch

    def _np(self, x):
        return x.numpy()

    def fft_rows(self, x, logn):
        y = orc.fft_forward(self._np(x).reshape(-1, 1 << logn))
        return self.torch.from_numpy(np.ascontiguousarray(y.reshape(-1)))

    def transpose(self, x, rows, cols):
        return self.torch.from_numpy(np.ascontiguousarray(self._np(x).reshape(rows, cols).T).reshape(-1))

    def twiddle_transpose(self, x, rows, cols, row0, col0, log_total):
        r = np.arange(rows)[:, None] + row0
        c = np.arange(cols)[None, :] + col0
        n = 1 << log_total
        w = np.exp(-2j * np.pi * ((r * c) % n) / n)
        return self.torch.from_numpy(np.ascontiguousarray((self._np(x).reshape(rows, cols) * w).T).reshape(-1))

    def permute102(self, x, a, b, run):
        return self.torch.from_numpy(np.ascontiguousarray(self._np(x).reshape(a, b, run).transpose(1, 0, 2)).reshape(-1))

    def all_to_all(self, x, group):
        import torch.distributed as dist

        out = self.torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cpu_worker(rank, world, port, logn, natural, q):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = 1 << logn
        x = orc.make_input(1, n, np.complex128, seed=42)[0]
        b, e = mg.shard_range(n, world, rank)
        fs = mg.FourStepFFT(logn, world, rank, HostBackend(torch), natural_order=natural)
        y = fs(torch.from_numpy(x[b:e].copy())).numpy()
        ref = orc.fft_forward(x)
        if natural:
            err = orc.rel_l2(y, ref[b:e])
        else:
            n1l = fs.n1 // world
            idx = np.array([[fs.output_index(k1, k2) for k2 in range(fs.n2)] for k1 in range(n1l)]).reshape(-1)
            err = orc.rel_l2(y, ref[idx])
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,logn,natural", [(2, 10, False), (2, 11, True), (4, 12, False), (4, 13, True)])
def test_four_step_distribution_logic_gloo(world, logn, natural):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_worker, args=(r, world, port, logn, natural, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert len(res) == world and all(e < 1e-12 for e in res.values()), res


def _mismatch_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        try:
            mg.FourStepFFT(10 + (rank == 1), world, rank, HostBackend(torch))   # rank 1 plans another length
            q.put((rank, "constructed"))
        except ValueError as e:
            q.put((rank, "refused: " + str(e)))
    finally:
        dist.destroy_process_group()


def test_mismatched_plans_are_refused_at_construction_gloo():
    """A rank that describes another transform than its peers is caught before any data moves:
    every rank raises at construction (nothing hangs, nothing is exchanged)."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_mismatch_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(2))
    assert all(v.startswith("refused") for v in res.values()), res


def _leaver_worker(rank, world, port, q):
    import datetime
    import time

    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    logn = 10
    n = 1 << logn
    x = orc.make_input(1, n, np.complex128, seed=1)[0]
    b, e = mg.shard_range(n, world, rank)
    fs = mg.FourStepFFT(logn, world, rank, HostBackend(torch))
    xl = torch.from_numpy(x[b:e].copy())
    fs(xl)                                   # step 1: everybody takes part
    def leave(msg):
        q.put((rank, msg))
        q.close()
        q.join_thread()                      # the message is on its way before the process goes
        os._exit(0)                          # (the process group cannot be torn down cleanly any more)

    if rank == world - 1:
        leave("left")                        # leaves between steps, nothing of its own in flight
    t0 = time.time()
    try:
        fs(xl)                               # step 2: one peer is gone
        msg = "completed"
    except Exception as ex:                  # noqa: BLE001 -- whatever the backend raises, it must raise
        msg = f"error after {time.time() - t0:.1f} s: {type(ex).__name__}"
    leave(msg)


def test_rank_that_leaves_between_steps_ends_the_others_with_an_error_gloo():
    """Failure detection without any device fault: a rank exits between two transforms; the
    remaining ranks' next exchange ends with an error inside the process-group timeout instead of
    hanging, so the caller can tear the job down."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 4
    procs = [ctx.Process(target=_leaver_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert p.exitcode is not None, "a rank hung after its peer left"
    res = dict(q.get(timeout=10) for _ in range(world))
    assert res[world - 1] == "left"
    assert all(res[r].startswith("error") for r in range(world - 1)), res


def test_batch_sharding_is_communication_free_gloo():
    """Each rank transforms its own contiguous batch range; concatenation equals the whole."""
    x = orc.make_input(10, 64, np.complex128, seed=3)
    parts = []
    for r in range(4):
        b, e = mg.shard_range(10, 4, r)
        parts.append(orc.fft_forward(x[b:e]))
    assert orc.rel_l2(np.concatenate(parts), orc.fft_forward(x)) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,logn,natural", [(0, 16, False), (0, 17, True), (1, 14, True), (1, 20, False)])
def test_four_step_kernels_single_gpu(torch_cuda, dtype, logn, natural):
    """World size 1: no exchange, but every local kernel of the four-step path runs."""
    torch = torch_cuda
    npdt = np.complex64 if dtype == 0 else np.complex128
    x = orc.make_input(1, 1 << logn, npdt, seed=logn)[0]
    fs = mg.FourStepFFT(logn, 1, 0, mg.DeviceBackend(dtype, 0), natural_order=natural)
    y = fs(torch.from_numpy(x).cuda()).cpu().numpy()
    ref = orc.fft_forward(x)
    if not natural:
        ref = ref.reshape(fs.n2, fs.n1).T.reshape(-1)   # [k1][k2]
    assert orc.rel_l2(y, ref) <= orc.tolerance(npdt, logn)


@pytest.mark.gpu
def test_helper_kernels(torch_cuda):
    import turbofft_b200 as tf

    torch = torch_cuda
    be = mg.DeviceBackend(1, 0)
    x = torch.randn(6 * 10 * 4, dtype=torch.complex128, device="cuda")
    assert torch.equal(be.permute102(x, 6, 10, 4).view(10, 6, 4), x.view(6, 10, 4).permute(1, 0, 2))
    assert torch.equal(be.transpose(x, 24, 10).view(10, 24), x.view(24, 10).t())
    t = be.twiddle_transpose(x, 24, 10, 5, 3, 12).view(10, 24).cpu().numpy()
    r = np.arange(24)[:, None] + 5
    c = np.arange(10)[None, :] + 3
    w = np.exp(-2j * np.pi * ((r * c) % 4096) / 4096)
    assert np.allclose(t, (x.view(24, 10).cpu().numpy() * w).T, atol=1e-13)
    src = torch.arange(1 << 20, dtype=torch.float32, device="cuda")
    dst = torch.zeros_like(src)
    tf.stream_copy(src, dst)
    assert torch.equal(src, dst)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,logn,natural", [(0, 16, False), (0, 19, True), (1, 14, True), (1, 18, False)])
def test_fused_four_step_single_gpu(torch_cuda, dtype, logn, natural):
    """World size 1: the fused scatter-transpose kernels store into this GPU's own buffers."""
    torch = torch_cuda
    npdt = np.complex64 if dtype == 0 else np.complex128
    x = orc.make_input(1, 1 << logn, npdt, seed=logn)[0]
    fs = mg.FusedFourStepFFT(logn, 1, 0, dtype, 0, natural_order=natural, if_ft=1, pipeline=2 if logn >= 16 else 1)
    y = fs(torch.from_numpy(x).cuda()).cpu().numpy()
    y2 = fs(torch.from_numpy(x).cuda()).cpu().numpy()     # buffers reused by a second call
    fs.close()
    ref = orc.fft_forward(x)
    if not natural:
        ref = ref.reshape(fs.n2, fs.n1).T.reshape(-1)
    assert orc.rel_l2(y, ref) <= orc.tolerance(npdt, logn)
    assert np.array_equal(y, y2)


def _gpu_worker(rank, world, port, logn, dtype, q):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        npdt = np.complex64 if dtype == 0 else np.complex128
        n = 1 << logn
        x = orc.make_input(1, n, npdt, seed=7)[0]
        b, e = mg.shard_range(n, world, rank)
        ref = orc.fft_forward(x)[b:e]
        fs = mg.FourStepFFT(logn, world, rank, mg.DeviceBackend(dtype, rank, if_ft=1), natural_order=True)
        y = fs(torch.from_numpy(x[b:e].copy()).cuda()).cpu().numpy()
        # the same transform with the exchanges fused into peer-storing kernels, twice in a row
        fused = mg.FusedFourStepFFT(logn, world, rank, dtype, rank, natural_order=True, if_ft=1)
        xg = torch.from_numpy(x[b:e].copy()).cuda()
        yf = fused(xg).cpu().numpy()
        yf2 = fused(xg).cpu().numpy()
        # natural order, calls back to back with NO host synchronisation in between: the copy-out of
        # call k reads the receive buffer that every peer's call k + 1 stores into first
        back = [fused(xg) for _ in range(4)]
        torch.cuda.synchronize()
        yf2 = max((t.cpu().numpy() for t in back), key=lambda a: orc.rel_l2(a, ref))
        dist.barrier()
        fused.close()
        # and with each exchange cut into pieces that overlap the local transforms
        piped = mg.FusedFourStepFFT(logn, world, rank, dtype, rank, natural_order=True, if_ft=1, pipeline=2)
        yp = piped(xg).cpu().numpy()
        yp2 = piped(xg).cpu().numpy()
        torch.cuda.synchronize()
        dist.barrier()
        piped.close()
        # and with the copy engines moving the packed pieces
        dma = mg.FusedFourStepFFT(logn, world, rank, dtype, rank, natural_order=True, if_ft=1, pipeline=2, exchange="dma")
        yd = dma(xg).cpu().numpy()
        yd2 = dma(xg).cpu().numpy()
        torch.cuda.synchronize()
        dist.barrier()
        dma.close()
        q.put((rank, max(orc.rel_l2(y, ref), orc.rel_l2(yf, ref), orc.rel_l2(yf2, ref), orc.rel_l2(yp, ref), orc.rel_l2(yp2, ref),
                         orc.rel_l2(yd, ref), orc.rel_l2(yd2, ref))))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,logn", [(0, 20), (1, 19)])
def test_four_step_two_gpus(torch_cuda, dtype, logn):
    torch = torch_cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, 2, port, logn, dtype, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(2))
    tol = orc.tolerance(np.complex64 if dtype == 0 else np.complex128, logn)
    assert all(e <= tol for e in res.values()), res


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,twiddle", [(0, 0), (0, 1), (1, 1)])
def test_pack_and_copy_exchange_single_gpu(torch_cuda, dtype, twiddle):
    """The copy-engine exchange on one device: two receivers, receiver 0 written directly (own share),
    receiver 1 through a packed send block and one 2-D copy; both must hold what the storing kernel
    leaves there, and that must be the numpy statement of the exchange."""
    import ctypes as C

    from turbofft_b200 import _lib
    from turbofft_b200._lib import lib

    torch = torch_cuda
    tdt = torch.complex64 if dtype == 0 else torch.complex128
    es = 8 if dtype == 0 else 16
    rows, cols, P, ld, row0, log_total = 64, 256, 2, 192, 64, 20
    cb = cols // P
    x = torch.randn(rows * cols, dtype=tdt, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # reference: the storing kernel into two receive buffers of pitch ld
    direct = [torch.zeros(cb * ld, dtype=tdt, device="cuda") for _ in range(P)]
    tab = (C.c_void_p * P)(*[d.data_ptr() for d in direct])
    _lib.check(lib().tfft_scatter_transpose_part(x.data_ptr(), tab, P, rows, cols, ld, row0, twiddle, log_total, 0, cb, 0,
                                                 dtype, stream), "tfft_scatter_transpose_part")
    # pack: receiver 0 in place, receiver 1 into a send block of pitch rows; then the 2-D copy, in two pieces
    recv = [torch.zeros(cb * ld, dtype=tdt, device="cuda") for _ in range(P)]
    send = torch.zeros(cb * rows, dtype=tdt, device="cuda")
    ptrs = (C.c_void_p * P)(recv[0].data_ptr(), send.data_ptr())
    lds = (C.c_longlong * P)(ld, rows)
    offs = (C.c_longlong * P)(row0, 0)
    for piece in range(2):
        sub = cb // 2
        _lib.check(lib().tfft_scatter_transpose_ex(x.data_ptr(), ptrs, lds, offs, P, rows, cols, row0, twiddle, log_total,
                                                   piece * sub, sub, 0, dtype, stream), "tfft_scatter_transpose_ex")
        _lib.check(lib().tfft_copy_2d(recv[1].data_ptr() + (piece * sub * ld + row0) * es, ld * es,
                                      send.data_ptr() + piece * sub * rows * es, rows * es, rows * es, sub, stream),
                   "tfft_copy_2d")
    torch.cuda.synchronize()
    for j in range(P):
        assert torch.equal(recv[j], direct[j])
    xm = x.view(rows, cols).cpu().numpy()
    if twiddle:
        r = np.arange(rows)[:, None] + row0
        c = np.arange(cols)[None, :]
        xm = xm * np.exp(-2j * np.pi * ((r * c) % (1 << log_total)) / (1 << log_total))
    for j in range(P):
        got = recv[j].view(cb, ld).cpu().numpy()[:, row0:row0 + rows]
        want = xm[:, j * cb:(j + 1) * cb].T
        assert np.abs(got - want).max() <= (2e-6 if dtype == 0 else 1e-14) * np.abs(want).max()
    # bad arguments are refused
    assert lib().tfft_copy_2d(None, 8, send.data_ptr(), 8, 8, 1, stream) != 0
    bad = (C.c_longlong * P)(rows - 1, rows)
    assert lib().tfft_scatter_transpose_ex(x.data_ptr(), ptrs, bad, offs, P, rows, cols, row0, twiddle, log_total, 0, cb, 0,
                                           dtype, stream) != 0


def test_dma_exchange_geometry_numpy():
    """The copy-engine exchange restated with numpy arrays for 4 ranks: pack per receiver, move every
    piece with the offsets dma_piece_geometry gives, and compare every receive buffer with the plain
    statement of the exchange (receiver j holds columns j*cb.. of everybody's rows, transposed)."""
    P, G = 4, 2
    n1, n2 = 64, 128                      # global matrix [n1][n2], rank r owns rows r*n1l..
    n1l, cb = n1 // P, n2 // P
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n1, n2)) + 1j * rng.standard_normal((n1, n2))
    recv = [np.zeros(cb * n1, dtype=complex) for _ in range(P)]          # [cb][ld = n1]
    for r in range(P):
        mine = x[r * n1l:(r + 1) * n1l]                                   # [rows][cols]
        rows, cols, ld, row0 = n1l, n2, n1, r * n1l
        send = np.concatenate([mine[:, j * cb:(j + 1) * cb].T.reshape(-1) for j in range(P)])   # [j][cb][rows]
        for g in range(G):
            for j in range(P):
                doff, dpitch, soff, spitch, width, height = mg.dma_piece_geometry(rows, cols, ld, row0, P, G, g, j)
                for h in range(height):
                    recv[j][doff + h * dpitch: doff + h * dpitch + width] = send[soff + h * spitch: soff + h * spitch + width]
    for j in range(P):
        assert np.array_equal(recv[j].reshape(cb, n1), x[:, j * cb:(j + 1) * cb].T)


def _split_parts(torch, x, devices):
    P = len(devices)
    n = x.shape[0]
    return [torch.from_numpy(x[r * n // P:(r + 1) * n // P].copy()).to(f"cuda:{d}") for r, d in enumerate(devices)]


def _check_single_process(torch, dtype, logn, devices, natural, pipeline, if_ft=0):
    npdt = np.complex64 if dtype == 0 else np.complex128
    x = orc.make_input(1, 1 << logn, npdt, seed=logn + len(devices))[0]
    fs = mg.SingleProcessFourStep(logn, dtype, devices, natural_order=natural, if_ft=if_ft, pipeline=pipeline)
    try:
        for _ in range(2):          # twice: the second call reuses the receive buffers behind the first
            outs = fs(_split_parts(torch, x, devices))
        y = np.concatenate([o.cpu().numpy() for o in outs])
        ref = orc.fft_forward(x)
        if not natural:
            ref = ref.reshape(1 << fs.l2, 1 << fs.l1).T.reshape(-1)     # [k1][k2], rows block-distributed over ranks
        assert orc.rel_l2(y, ref) <= orc.tolerance(npdt, logn)
        if if_ft:
            assert fs.ft_counts() == (0, 0)
    finally:
        fs.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,logn,ranks,natural,pipeline", [(0, 16, 1, False, 1), (1, 14, 1, True, 2), (0, 18, 2, False, 1),
                                                              (0, 18, 2, True, 2), (1, 17, 4, False, 1), (0, 20, 4, True, 2),
                                                              (1, 16, 2, False, 2)])
def test_single_process_four_step_ranks_on_one_gpu(torch_cuda, dtype, logn, ranks, natural, pipeline):
    """tfft_mg_* with every rank on device 0: the whole exchange / event logic of the multi-device
    plan runs on one GPU (nothing in it waits on a peer, so ranks may share a device)."""
    _check_single_process(torch_cuda, dtype, logn, [0] * ranks, natural, pipeline, if_ft=int(logn == 18))


@pytest.mark.gpu
def test_single_process_four_step_refuses_bad_plans(torch_cuda):
    import ctypes as C

    import turbofft_b200 as tf

    lib = tf.lib()
    h = C.c_void_p()
    dev = (C.c_int * 4)(0, 0, 0, 0)
    assert lib.tfft_mg_plan_create(C.byref(h), 20, 0, 0, 3, dev, 0, 1) == -1       # ranks not a power of two
    assert lib.tfft_mg_plan_create(C.byref(h), 14, 0, 0, 4, dev, 0, 2) == -2       # shares too small for 2 pieces of 32 lines
    assert lib.tfft_mg_plan_create(C.byref(h), 20, 7, 0, 2, dev, 0, 1) == -1       # no such datatype


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,logn,natural,pipeline", [(0, 22, False, 4), (1, 20, True, 2)])
def test_single_process_four_step_two_gpus(torch_cuda, dtype, logn, natural, pipeline):
    if torch_cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _check_single_process(torch_cuda, dtype, logn, [0, 1], natural, pipeline, if_ft=1)
