"""Row-partitioned SpMV / SpMM / PCG over the GPUs of one node, one process per GPU.

``torch.distributed`` carries the plumbing (NCCL over NVLink on GPUs; gloo in the
CPU tests of the host logic).  The data path has an exchange only where the
operator needs one:

* SpMV / SpMM: rank g owns an nnz-balanced block of rows; x (or B) is replicated, as
  a caller that holds the same right-hand side on every GPU has it; no collective.
* PCG: every vector is split like the rows.  Before the SpMV pass each rank needs the
  pieces of p that its columns reach outside its own block (for a banded matrix one
  grid row from each neighbour), and the two scalar groups of an iteration (p.Ap; r.r
  and r.z) must be summed over the ranks.  Two transports: ``comm="p2p"`` (default on
  several GPUs) -- every rank maps its peers' workspaces and mailboxes with CUDA IPC,
  the producers store straight into peer memory over NVLink and raise sequence-numbered
  flags, small kernels wait for them with a bound; ``comm="nccl"`` -- NCCL send/recv
  for the halo and two allreduces of the solver's scalar block.  One iteration is
  captured in a CUDA graph and replayed, so the host is not in the loop between checks
  of the stop flag.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import partition as part


class HaloExchanger:
    """Moves the non-owned pieces of a window [c0, c1) of a row-distributed vector.

    ``ext`` passed to :meth:`exchange` is this rank's window buffer: element i holds
    global entry c0 + i; the owned entries [r0, r1) must be current on entry, the rest is
    overwritten with the owners' values.
    """

    def __init__(self, bounds, windows, rank: int, group=None):
        self.rank = rank
        self.group = group
        self.bounds = np.asarray(bounds, dtype=np.int64)
        self.c0, self.c1 = windows[rank]
        self.r0, self.r1 = int(self.bounds[rank]), int(self.bounds[rank + 1])
        recv, send = part.exchange_plan(self.bounds, windows)
        self.recv, self.send = recv[rank], send[rank]

    @property
    def own_offset(self) -> int:
        return self.r0 - self.c0

    @property
    def window_len(self) -> int:
        return self.c1 - self.c0

    def exchange(self, ext: torch.Tensor) -> None:
        if not self.recv and not self.send:
            return
        ops = []
        # Every rank lists its transfers by ascending peer, sends and receives interleaved the
        # same way on both sides, so that batched point-to-point calls pair up.
        peers = sorted({p for p, _, _ in self.recv} | {p for p, _, _ in self.send})
        for peer in peers:
            for (p, s, e) in self.send:
                if p == peer:
                    ops.append(dist.P2POp(dist.isend, ext[s - self.c0:e - self.c0], self._global_rank(peer), self.group))
            for (p, s, e) in self.recv:
                if p == peer:
                    ops.append(dist.P2POp(dist.irecv, ext[s - self.c0:e - self.c0], self._global_rank(peer), self.group))
        for req in dist.batch_isend_irecv(ops):
            req.wait()

    def _global_rank(self, group_rank: int) -> int:
        return group_rank if self.group is None else dist.get_global_rank(self.group, group_rank)


def local_block(pos, crd, val, rank: int, world: int):
    """This rank's row block of a host CSR: (bounds, local pos, crd, val)."""
    bounds = part.partition_rows(pos, world)
    lpos, lcrd, lval = part.row_block(pos, crd, val, int(bounds[rank]), int(bounds[rank + 1]))
    return bounds, lpos, lcrd, lval


def all_windows(pos, crd, bounds):
    """Column window of every rank (each rank can compute all of them from the host CSR)."""
    wins = []
    for g in range(len(bounds) - 1):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        wins.append(part.column_window(crd[int(pos[r0]):int(pos[r1])], r0, r1))
    return wins


class ShardedSpmv:
    """y_local = (y_local) + A[rows of this rank, :] x with x replicated on every rank."""

    def __init__(self, pos, crd, val, shape, rank: int, world: int, device, tune="strict"):
        from .device import CsrMatrix
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.ncols = int(shape[1])
        self.bounds, lpos, lcrd, lval = local_block(pos, crd, val, rank, world)
        self.r0, self.r1 = int(self.bounds[rank]), int(self.bounds[rank + 1])
        self.matrix = CsrMatrix.from_host(lpos, lcrd, lval, (self.r1 - self.r0, shape[1]), device, tune=tune == "strict")
        if tune == "relaxed":
            self.matrix.tune(relaxed=True)
        self._x = None
        self._y = None

    def spmv(self, x, y_local, accumulate=True):
        return self.matrix.spmv(x, y_local, accumulate)

    def spmm(self, B, C_local, accumulate=True):
        return self.matrix.spmm(B, C_local, accumulate)

    def spmv_from_host(self, x_host: torch.Tensor, y_host_local: torch.Tensor, group=None):
        """y_local = A[rows of this rank, :] x with x and y in (page-locked) host memory: every rank uploads only
        its 1/world slice of x, the slices are gathered over NVLink into the full x on every GPU (NCCL
        all-gather; with one rank the whole x is uploaded), the kernel runs, and this rank's block of y is
        copied back.  Returns when y_host_local is current.  Uploading all of x from the one host on every
        rank instead costs world times the PCIe traffic for the same result."""
        n = self.ncols
        if self._x is None:
            self._x = torch.empty(n, dtype=torch.float64, device=self.device)
            self._y = torch.empty(self.r1 - self.r0, dtype=torch.float64, device=self.device)
        if self.world > 1 and n % self.world == 0:
            per = n // self.world
            if getattr(self, "_x_slice", None) is None:
                self._x_slice = torch.empty(per, dtype=torch.float64, device=self.device)
            self._x_slice.copy_(x_host[self.rank * per:(self.rank + 1) * per], non_blocking=True)
            dist.all_gather_into_tensor(self._x, self._x_slice, group=group)
        else:
            self._x.copy_(x_host, non_blocking=True)
        self.matrix.spmv(self._x, self._y, accumulate=False)
        y_host_local.copy_(self._y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return y_host_local


class _PeerBuffer:
    """Device memory from ``lapis_b200_peer_alloc``: zero-initialised, exportable as a CUDA IPC handle,
    visible to torch as a float64 tensor (zero-copy) through ``__cuda_array_interface__``."""

    def __init__(self, lib, check, nbytes: int, device):
        self._lib, self._check = lib, check
        self.nbytes = int(nbytes)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            check(lib.lapis_b200_peer_alloc(self.nbytes, ctypes.byref(ptr), handle))
        self.ptr, self.handle = int(ptr.value), handle.raw
        self.__cuda_array_interface__ = {"shape": (self.nbytes // 8,), "typestr": "<f8", "data": (self.ptr, False),
                                         "version": 2, "strides": None}
        self.tensor = torch.as_tensor(self, device=device)

    def free(self):
        if self.ptr:
            self.tensor = None
            self._lib.lapis_b200_peer_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


class DistPcg:
    """Jacobi-preconditioned CG (examples/pcg_solve.py:52-101 in the LAPIS project) on a
    row-partitioned matrix.  Construct on every rank with the same host CSR, b and dinv."""

    GRAPH_UNROLL = 5  # iterations per launch of the larger of the two captured graphs

    def __init__(self, pos, crd, val, shape, b, dinv, device, group=None, use_graph: bool = True, comm: str = "p2p",
                 transport_on_one_rank: bool = False, tune: bool = True, fused: bool = True, two_pass: bool = True):
        from ._lib import check, load
        from .device import CsrMatrix
        self._check, self._lib = check, load()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = torch.device(device)
        self.use_graph = use_graph
        # fused: one iteration is three launches (sums and exchanges inside the passes); False keeps the
        # older form with separate summing / exchange kernels between the passes
        self.fused = fused
        # two_pass: fold the direction update into the next SpMV pass where the matrix allows it (two launches)
        self.two_pass = two_pass
        n_global = int(shape[0])
        if shape[0] != shape[1]:
            raise ValueError("pcg: matrix is not square")
        self.bounds, lpos, lcrd, lval = local_block(pos, crd, val, self.rank, self.world)
        windows = all_windows(pos, crd, self.bounds)
        self.halo = HaloExchanger(self.bounds, windows, self.rank, group)
        self.n = self.halo.r1 - self.halo.r0
        self.n_p = self.halo.window_len
        self.p_off = self.halo.own_offset
        lcrd = (lcrd.astype(np.int64) - self.halo.c0).astype(lcrd.dtype)  # columns index the window
        with torch.cuda.device(self.device):
            self.matrix = CsrMatrix.from_host(lpos, lcrd, lval, (self.n, self.n_p), self.device, tune=tune)
            sl = slice(self.halo.r0, self.halo.r1)
            self.b = torch.as_tensor(np.ascontiguousarray(b[sl])).to(self.device)
            self.dinv = torch.as_tensor(np.ascontiguousarray(dinv[sl])).to(self.device)
            self.x = torch.zeros(self.n, dtype=torch.float64, device=self.device)
            nbytes = int(self._lib.lapis_b200_pcg_workspace_bytes(self.n, self.n_p))
            if comm not in ("p2p", "nccl"):
                raise ValueError("comm must be 'p2p' or 'nccl'")
            # one rank needs no exchange; transport_on_one_rank keeps the peer-to-peer kernels in the loop
            # anyway (the rank is its own only peer), which exercises them on a single GPU
            self.comm = comm if self.world > 1 or (transport_on_one_rank and comm == "p2p") else "none"
            if self.comm == "p2p":
                self._work_buf = _PeerBuffer(self._lib, check, nbytes, self.device)
                self.work = self._work_buf.tensor
            else:
                self.work = torch.zeros(nbytes // 8, dtype=torch.float64, device=self.device)
            offs = (ctypes.c_int64 * 4)()
            check(self._lib.lapis_b200_pcg_workspace_layout(self.n, self.n_p, offs))
            self._p_doubles = int(offs[2])
            self._zh_doubles = int(offs[3]) + self.n   # the z halo buffer follows Ap
            self.p_ext = self.work[offs[2]:offs[2] + self.n_p]
            self.sc = self.work[0:8]
            self.flags = self.work[8:10].view(torch.int64)
            if self.comm == "p2p":
                self._setup_p2p(windows)
        self.n_global = n_global
        self._graph = None
        self._epoch = 0

    # -- peer-to-peer transport -----------------------------------------------------------
    def _setup_p2p(self, windows):
        """Exchanges IPC handles, maps every peer's workspace and mailbox, and builds the device tables
        the exchange kernels read: mailbox addresses, halo pieces to push, ranks to wait for."""
        lib, check = self._lib, self._check
        if self.world > 16:
            raise ValueError("the peer-to-peer transport supports up to 16 ranks")
        self._mbox_buf = _PeerBuffer(lib, check, int(lib.lapis_b200_pcg_p2p_mailbox_bytes()), self.device)
        mine = (self._work_buf.handle, self._mbox_buf.handle, self.n_p, self._p_doubles, self._zh_doubles)
        infos = [mine] * self.world
        if self.world > 1:
            dist.all_gather_object(infos, mine, group=self.group)
        self._peer_ptrs = []
        work_addr, mbox_addr = [0] * self.world, [0] * self.world
        for r, (wh, mh, _, _, _) in enumerate(infos):
            if r == self.rank:
                work_addr[r], mbox_addr[r] = self._work_buf.ptr, self._mbox_buf.ptr
                continue
            for h, table in ((wh, work_addr), (mh, mbox_addr)):
                ptr = ctypes.c_void_p()
                check(lib.lapis_b200_peer_open(h, ctypes.byref(ptr)))
                table[r] = int(ptr.value)
                self._peer_ptrs.append(int(ptr.value))
        self._peer_mbox = torch.tensor(mbox_addr, dtype=torch.int64, device=self.device)
        halo_index, err_index = ctypes.c_int64(), ctypes.c_int64()
        lib.lapis_b200_pcg_p2p_mailbox_layout(ctypes.byref(halo_index), ctypes.byref(err_index))
        HALO, self._err_index = int(halo_index.value), int(err_index.value)
        pieces = part.push_pieces(self.halo.send, windows, self.rank, [i[2] for i in infos], [i[3] for i in infos],
                                  work_addr, mbox_addr, HALO)
        self._npieces = len(pieces) // 4
        # the same pieces aimed at the neighbours' z halo buffers (fused passes), and the halo parts of this
        # rank's own window, which pass C updates from those buffers
        zpieces = part.push_pieces(self.halo.send, windows, self.rank, [i[2] for i in infos], [i[4] for i in infos],
                                   work_addr, mbox_addr, HALO)
        self._nzpieces = len(zpieces) // 4
        self._zpieces = torch.tensor(zpieces if zpieces else [0], dtype=torch.int64, device=self.device)
        ranges = []
        for (_, s0, e0) in sorted(self.halo.recv, key=lambda t: t[1]):
            ranges += [s0 - self.halo.c0, e0 - s0]
        self._nranges = len(ranges) // 2
        self._halo_ranges = torch.tensor(ranges if ranges else [0], dtype=torch.int64, device=self.device)
        self._nsrc_fused = 0
        self._pieces = torch.tensor(pieces if pieces else [0], dtype=torch.int64, device=self.device)
        srcs = sorted({owner for owner, _, _ in self.halo.recv})
        self._nsrc = len(srcs)
        self._srcs = torch.tensor(srcs if srcs else [0], dtype=torch.int32, device=self.device)
        # the fused passes keep at most 32 halo pieces in shared memory and poll at most 32 sources; the ranks
        # decide together, so that all of them run the same form of the iteration
        fits = [self._nzpieces <= 32 and self._nsrc <= 32] * self.world
        if self.world > 1:
            dist.all_gather_object(fits, fits[0], group=self.group)
        self.fused = self.fused and all(fits)
        if self.world > 1:
            dist.barrier(group=self.group)  # every rank has mapped every buffer before anyone pushes

    def _p2p_scalars(self, phase: int, derive: int, tol: float, maxiter: int):
        lib, check, w = self._lib, self._check, ctypes.c_void_p(self.work.data_ptr())
        check(lib.lapis_b200_pcg_p2p_push_scalars(w, phase, self.rank, self.world,
                                                  ctypes.c_void_p(self._peer_mbox.data_ptr()), self._stream()))
        check(lib.lapis_b200_pcg_p2p_wait_reduce(w, ctypes.c_void_p(self._mbox_buf.ptr), phase, self.world, derive, tol,
                                                 maxiter, self._stream()))

    def _p2p_halo_push(self):
        self._check(self._lib.lapis_b200_pcg_p2p_halo_push(ctypes.c_void_p(self.work.data_ptr()), self.n, self.n_p,
                                                           ctypes.c_void_p(self._pieces.data_ptr()), self._npieces,
                                                           self._stream()))

    def _p2p_halo_wait(self):
        self._check(self._lib.lapis_b200_pcg_p2p_halo_wait(ctypes.c_void_p(self.work.data_ptr()),
                                                           ctypes.c_void_p(self._mbox_buf.ptr),
                                                           ctypes.c_void_p(self._srcs.data_ptr()), self._nsrc, self._stream()))

    def comm_error(self) -> float:
        """Non-zero when a bounded wait of the peer-to-peer transport gave up (1-3: scalars, 9: halo)."""
        return float(self._mbox_buf.tensor[self._err_index].item()) if self.comm == "p2p" else 0.0

    # -- one iteration, enqueued on the current stream ---------------------------------
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _allreduce(self, t):
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def _exchange(self):
        """The exchange description the fused passes take (NULL on one rank without the transport)."""
        if self.comm != "p2p":
            return None
        ex = getattr(self, "_exchange_struct", None)
        if ex is None:
            from ._lib import PcgExchange
            # no halo flags to wait for in the steady state (_nsrc_fused == 0): the halo of p is recomputed from the
            # neighbours' rows of z; the halo of the first p is waited for once, after the initialisation
            ex = PcgExchange(self.rank, self.world, ctypes.c_void_p(self._mbox_buf.ptr),
                             ctypes.c_void_p(self._peer_mbox.data_ptr()), ctypes.c_void_p(self._srcs.data_ptr()),
                             self._nsrc_fused, ctypes.c_void_p(self._zpieces.data_ptr()), self._nzpieces,
                             ctypes.c_void_p(self._halo_ranges.data_ptr()), self._nranges)
            self._exchange_struct = ex
        return ctypes.byref(ex)

    def _two_pass(self) -> bool:
        """Whether an iteration is two launches (matrices served by the one-thread-per-row SpMV kernel)."""
        tp = getattr(self, "_two_pass_cached", None)
        if tp is None:
            tp = bool(self.two_pass and self.fused and self.comm in ("p2p", "none")
                      and self._lib.lapis_b200_pcg_folds_direction(self.matrix.handle))
            self._two_pass_cached = tp
        return tp

    def _iteration(self, tol: float, maxiter: int):
        lib, check, w = self._lib, self._check, ctypes.c_void_p(self.work.data_ptr())
        if self.fused and self.comm in ("p2p", "none"):
            # three launches: the sums are added in the last block of each pass and, with the peer-to-peer
            # transport, the exchanges happen inside the passes
            ex = self._exchange()
            if self._two_pass():
                # two launches: the direction update of the iteration before is folded into the SpMV pass
                check(lib.lapis_b200_pcg_fused_spmv_direction(w, self.matrix.handle, self.n_p, self.p_off, tol, maxiter, ex,
                                                              self._stream()))
            else:
                check(lib.lapis_b200_pcg_fused_spmv(w, self.matrix.handle, self.n_p, self.p_off, tol, maxiter, ex, self._stream()))
            check(lib.lapis_b200_pcg_fused_update(w, self.n, self.n_p, self.p_off, ctypes.c_void_p(self.dinv.data_ptr()),
                                                  ctypes.c_void_p(self.x.data_ptr()), tol, maxiter, ex, self._stream()))
            if not self._two_pass():
                check(lib.lapis_b200_pcg_fused_direction(w, self.n, self.n_p, self.p_off, tol, maxiter, ex, self._stream()))
            return
        single = 1 if self.comm == "none" else 0
        p2p = self.comm == "p2p"
        if p2p:
            self._p2p_halo_wait()
        elif self.world > 1:
            self.halo.exchange(self.p_ext)
        check(lib.lapis_b200_pcg_step_spmv(w, self.matrix.handle, self.n_p, self.p_off, single, self._stream()))
        if p2p:
            self._p2p_scalars(0, 2, tol, maxiter)
        elif not single:
            self._allreduce(self.sc[0:1])
            check(lib.lapis_b200_pcg_derive(w, 2, tol, maxiter, self._stream()))
        check(lib.lapis_b200_pcg_step_update(w, self.n, self.n_p, self.p_off, ctypes.c_void_p(self.dinv.data_ptr()),
                                             ctypes.c_void_p(self.x.data_ptr()), single, tol, maxiter, self._stream()))
        if p2p:
            self._p2p_scalars(1, 3, tol, maxiter)
        elif not single:
            self._allreduce(self.sc[1:3])
            check(lib.lapis_b200_pcg_derive(w, 3, tol, maxiter, self._stream()))
        check(lib.lapis_b200_pcg_step_direction(w, self.n, self.n_p, self.p_off, self._stream()))
        if p2p:
            self._p2p_halo_push()

    def _init(self, tol, maxiter):
        lib, check, w = self._lib, self._check, ctypes.c_void_p(self.work.data_ptr())
        single = 1 if self.comm == "none" else 0
        check(lib.lapis_b200_pcg_init(w, self.n, self.n_p, self.p_off, ctypes.c_void_p(self.b.data_ptr()),
                                      ctypes.c_void_p(self.dinv.data_ptr()), ctypes.c_void_p(self.x.data_ptr()),
                                      single, self._stream()))
        if self.comm == "p2p":
            # a new epoch per solve: sequence numbers left in the mailboxes by an earlier solve never match
            self._epoch += 1
            self.work[10:11].fill_(float(self._epoch) * 4294967296.0)
            self._p2p_scalars(2, 1, tol, maxiter)
            self._p2p_halo_push()
            if self.fused:
                self._p2p_halo_wait()  # the halo of the first p; later halos are recomputed inside pass C
        elif not single:
            self._allreduce(self.sc[1:3])
            check(lib.lapis_b200_pcg_derive(w, 1, tol, maxiter, self._stream()))

    def solve(self, tol: float, maxiter: int, check_every: int = 25):
        """Returns (x_local, iters, relres); x_local holds rows [bounds[rank], bounds[rank+1])."""
        limit = maxiter if maxiter > 0 else 1 << 31
        with torch.cuda.device(self.device):
            if self.comm == "p2p" and self.world > 1:
                # the waits of the exchange kernels are bounded (seconds): start the ranks together
                dist.barrier(group=self.group)
            self._init(tol, maxiter)
            if self.use_graph and self._graph is None:
                # Warm up once on a side stream (NCCL and the kernels must have run before capture);
                # then rewind the solver state and capture one iteration.
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._iteration(tol, maxiter)
                torch.cuda.current_stream().wait_stream(s)
                torch.cuda.synchronize()
                self._init(tol, maxiter)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._iteration(tol, maxiter)
                # the same iteration GRAPH_UNROLL times in one graph: a graph launch costs more on the device than the
                # step from one kernel to the next inside a graph, which shows once a rank's share is small
                gk = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gk):
                    for _ in range(self.GRAPH_UNROLL):
                        self._iteration(tol, maxiter)
                self._graph = (g, tol, maxiter, gk)
                self._init(tol, maxiter)  # capture does not execute; state is still the initial one
            # the captured iteration has its tol / maxiter baked in: other values run as plain launches
            replay = self._graph is not None and self._graph[1:3] == (tol, maxiter)
            i = 0
            done = False
            while not done and i < limit:
                burst = min(check_every, limit - i)
                if replay:
                    for _ in range(burst // self.GRAPH_UNROLL):
                        self._graph[3].replay()
                    for _ in range(burst % self.GRAPH_UNROLL):
                        self._graph[0].replay()
                else:
                    for _ in range(burst):
                        self._iteration(tol, maxiter)
                i += burst
                fl = self.flags.cpu()
                done = bool(fl[0].item())
            if not done and self.comm == "p2p" and self._two_pass():
                # with an exchange the stop test of an iteration runs at the head of the next SpMV pass: one more
                # (it stops there: the iteration count has reached maxiter)
                self._check(self._lib.lapis_b200_pcg_fused_spmv_direction(
                    ctypes.c_void_p(self.work.data_ptr()), self.matrix.handle, self.n_p, self.p_off, tol, maxiter,
                    self._exchange(), self._stream()))
            iters = int(self.flags[1].item())
            relres = float(self.sc[5].item())
            err = self.comm_error()
            if err != 0.0:
                raise RuntimeError(f"pcg: a peer did not deliver in time (exchange {int(err)}: 1-3 scalar sums, 9 halo)")
            # a persistent SpMV block whose bounded wait gave up leaves Ap incomplete: the solve is not valid then
            self._check(self._lib.lapis_b200_spmv_status(self._stream()))
        return self.x, iters, relres
