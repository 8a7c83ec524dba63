"""Communicator: the Python face of the native context (``csrc/comm/comm.cu``).

One process drives one GPU.  Under ``torchrun`` (``torch.distributed`` initialised) the communicator
spans all processes and maps every peer's symmetric heap through CUDA IPC; the handles travel over a
gloo side group, so NCCL is not needed for bootstrap.  Without ``torch.distributed`` the communicator
lives in one process and hosts all ``nranks`` logical ranks on one GPU.

It replaces what ``MPI_Init`` / ``MPI_Comm`` / ``MPI_Comm_split`` are to the reference: ranks, groups and
the transport (peer stores over NVLink instead of MPI point-to-point).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np
import torch

from .. import _native
from .._cuda_decl import SITE_NAMES, STATUS_NAMES, Status
from .plan import ALGO_ID, Plan

_default_comm: Optional["Communicator"] = None


class CommError(RuntimeError):
    pass


class _Block:
    """Owner of one symmetric-heap allocation, exposed to torch through the CUDA array interface."""

    def __init__(self, comm: "Communicator", nbytes: int):
        self._comm = comm
        self.nbytes = int(nbytes)
        self.ptr = comm._lib.rbv_symm_alloc(comm._ctx, max(self.nbytes, 1))
        if not self.ptr:
            raise MemoryError(f"symmetric heap exhausted while allocating {nbytes} bytes "
                              f"(heap_bytes={comm.heap_bytes})")
        self.__cuda_array_interface__ = {"shape": (max(self.nbytes, 1),), "typestr": "|u1",
                                         "data": (self.ptr, False), "version": 3, "strides": None}

    def __del__(self):
        comm = getattr(self, "_comm", None)
        if comm is not None and getattr(comm, "_ctx", None) and getattr(self, "ptr", None):
            comm._lib.rbv_symm_free(comm._ctx, C.c_void_p(self.ptr))
            self.ptr = None


class PreparedCall:
    """A resolved collective; see :meth:`Communicator.prepare`."""

    KINDS = {0: "rendezvous", 1: "eager", 2: "static"}

    def __init__(self, comm: "Communicator", handle, keep, mirrored=None):
        self._comm, self._h, self._keep = comm, C.c_void_p(handle), keep
        self._mirrored = mirrored or []      # (caller's tensor, symmetric stand-in) pairs, see Communicator.prepare
        self._launch = comm._lib.rbv_launch
        self._ctx = comm._ctx
        self._dev = comm.device
        info = (C.c_longlong * 3)()
        #: which kernel runs the call: "static" (all counts resolved on the host, no metadata phase),
        #: "rendezvous" (metadata exchanged by the kernel) or "eager"
        self.kind = self.KINDS[comm._lib.rbv_prepared_info(self._h, info)]
        self.grid, self.cooperative, self.items = int(info[0]), bool(info[1]), int(info[2])

    def launch(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        st = stream or torch.cuda.current_stream(self._dev)
        rc = self._launch(self._ctx, self._h, C.c_void_p(st.cuda_stream))
        if rc:
            raise CommError("launch failed: " + self._comm._lib.rbv_last_error().decode())
        if self._mirrored and self.kind != "static":     # the static kernel has copied them on itself
            with torch.cuda.stream(st):
                for t, bt in self._mirrored:
                    t.reshape(-1).view(torch.uint8).copy_(bt, non_blocking=True)

    __call__ = launch

    def __del__(self):
        comm, h = getattr(self, "_comm", None), getattr(self, "_h", None)
        if comm is not None and h and getattr(comm, "_ctx", None):
            comm._lib.rbv_prepared_free(comm._ctx, h)
            self._h = None


class Communicator:
    def __init__(self, nranks: Optional[int] = None, device: Optional[int] = None,
                 heap_bytes: int = 1 << 30, arena_bytes: int = 32 << 20, timeout_ms: float = 2000.0):
        import torch.distributed as dist

        self._lib = _native.cuda_lib()
        self._dist = dist if dist.is_available() and dist.is_initialized() else None
        if self._dist is not None:
            self.nproc = dist.get_world_size()
            self.proc = dist.get_rank()
        else:
            self.nproc, self.proc = 1, 0
        if device is None:
            device = int(os.environ.get("LOCAL_RANK", "0")) if self._dist is not None else torch.cuda.current_device()
        self.device = int(device)
        torch.cuda.set_device(self.device)
        self.P = int(nranks) if nranks else self.nproc
        if self.P % self.nproc:
            raise ValueError(f"nranks={self.P} is not a multiple of the process count {self.nproc}")
        self.L = self.P // self.nproc
        self.heap_bytes = int(heap_bytes)
        self.arena_bytes = int(arena_bytes)
        torch.zeros(1, device=f"cuda:{self.device}")  # make sure the primary context exists
        self._ctx = C.c_void_p(self._lib.rbv_ctx_create(self.P, self.nproc, self.proc, self.device,
                                                        self.heap_bytes, self.arena_bytes))
        if not self._ctx:
            raise CommError("context creation failed: " + self._lib.rbv_last_error().decode())
        self._lib.rbv_ctx_set_timeout_ms(self._ctx, float(timeout_ms))
        self._bulk = int(os.environ.get("RBV_BULK", "0"))
        self._side = None
        if self.nproc > 1:
            self._side = dist.new_group(backend="gloo")
            mine = (C.c_char * 64)()
            rc = self._lib.rbv_ctx_ipc_handle(self._ctx, mine)
            if rc:
                raise CommError("cudaIpcGetMemHandle failed: " + self._lib.rbv_last_error().decode())
            handles = [None] * self.nproc
            dist.all_gather_object(handles, bytes(mine.raw), group=self._side)
            blob = b"".join(handles)
            rc = self._lib.rbv_ctx_connect(self._ctx, blob)
            if rc:
                raise CommError("cudaIpcOpenMemHandle failed: " + self._lib.rbv_last_error().decode())
            dist.barrier(group=self._side)
        self.nvls = False
        self.nvls_owner = None
        if self.nproc > 1 and os.environ.get("RBV_NVLS", "0") in ("1", "torch"):
            self._enable_nvls()
        info = (C.c_longlong * 8)()
        self._lib.rbv_ctx_info(self._ctx, info)
        self.max_ctas = int(info[6])
        self.sm_count = int(info[7])

    def _enable_nvls(self) -> None:
        """Moves the metadata tables into a buffer bound to an NVLink multicast object, so that the metadata phase
        publishes with ``multimem.st`` (NVSwitch replicates one store into the tables of all GPUs) and the auxiliary
        barriers arrive with one ``multimem.red``.  The object is the library's own: process 0 creates it with the
        CUDA driver API and hands its file descriptor to the other processes over a Unix socket (``SCM_RIGHTS``);
        every process adds its device, binds a buffer of its own and maps both views (``csrc/comm/comm.cu``,
        ``Context::nvls_*``).  ``RBV_NVLS=torch`` borrows torch's symmetric-memory allocator for the object instead.
        Opt-in (``RBV_NVLS=1``) and kept off in fault tests: a process that dies while its memory is bound to a
        multicast object disturbs the other GPUs."""
        if os.environ.get("RBV_NVLS") == "torch":
            return self._enable_nvls_torch()
        import socket
        import tempfile
        lib, dist = self._lib, self._dist
        nbytes = max(int(lib.rbv_ctx_meta_bytes(self._ctx)), 4096)

        def agree(ok: bool) -> bool:
            if not ok and os.environ.get("RBV_VERBOSE"):
                print(f"[rbv nvls, process {self.proc}] " + lib.rbv_last_error().decode(), flush=True)
            flag = torch.tensor([1 if ok else 0], dtype=torch.int64)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self._side)
            return bool(int(flag.item()))

        # step 1: process 0 creates the object; the descriptor travels over a Unix socket
        fd, size, ok, srv, path = C.c_int(-1), C.c_size_t(0), True, None, None
        if self.proc == 0:
            ok = lib.rbv_ctx_nvls_create(self._ctx, nbytes, C.byref(fd), C.byref(size)) == 0
            if ok:
                path = os.path.join(tempfile.mkdtemp(prefix="rbv_nvls_"), "fd.sock")
                srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                srv.bind(path)
                srv.listen(self.nproc)
        info = [(path, int(size.value)) if self.proc == 0 else None]
        dist.broadcast_object_list(info, src=0, group=self._side)
        path, obj_bytes = info[0]
        if not agree(ok and path is not None):
            if srv is not None:
                srv.close()
            lib.rbv_ctx_nvls_teardown(self._ctx)
            return
        if self.proc == 0:
            for _ in range(self.nproc - 1):
                conn, _ = srv.accept()
                socket.send_fds(conn, [b"fd"], [fd.value])
                conn.close()
            srv.close()
            os.close(fd.value)
            try:
                os.unlink(path)
                os.rmdir(os.path.dirname(path))
            except OSError:
                pass
        else:
            cli = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            cli.connect(path)
            _, fds, _, _ = socket.recv_fds(cli, 16, 1)
            cli.close()
            ok = lib.rbv_ctx_nvls_import(self._ctx, fds[0], obj_bytes) == 0
            os.close(fds[0])
        # steps 2-4, each completed everywhere before the next starts
        for step in (lib.rbv_ctx_nvls_add_device, lib.rbv_ctx_nvls_bind):
            ok = agree(ok) and step(self._ctx) == 0
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self._side)
        if not agree(ok):
            lib.rbv_ctx_nvls_teardown(self._ctx)
            return
        self.nvls = True
        self.nvls_owner = "library"

    def _enable_nvls_torch(self) -> None:
        """The same with a multicast object created and bound by torch's symmetric-memory allocator."""
        try:
            import torch.distributed._symmetric_memory as symm
            nbytes = max(int(self._lib.rbv_ctx_meta_bytes(self._ctx)), 4096)
            buf = symm.empty(nbytes, dtype=torch.uint8, device=f"cuda:{self.device}")
            hdl = symm.rendezvous(buf, group=self._dist.group.WORLD)
            mc = int(hdl.multicast_ptr) if hdl.has_multicast_support else 0
        except Exception:   # no multicast support on this system / build
            mc, buf, hdl = 0, None, None
        flag = torch.tensor([1 if mc else 0], dtype=torch.int64)
        self._dist.all_reduce(flag, op=self._dist.ReduceOp.MIN, group=self._side)
        if int(flag.item()) == 0:
            return
        buf.zero_()
        torch.cuda.synchronize(self.device)
        self._dist.barrier(group=self._side)
        rc = self._lib.rbv_ctx_set_nvls_meta(self._ctx, C.c_void_p(buf.data_ptr()), C.c_void_p(mc), nbytes)
        if rc:
            raise CommError("NVLS metadata setup failed: " + self._lib.rbv_last_error().decode())
        torch.cuda.synchronize(self.device)
        self._dist.barrier(group=self._side)
        self._nvls_keep = (buf, hdl)
        self.nvls = True
        self.nvls_owner = "torch"

    # ---- life cycle -------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_ctx", None):
            torch.cuda.synchronize(self.device)
            if self._side is not None:
                self._dist.barrier(group=self._side)
            self._lib.rbv_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            if getattr(self, "_ctx", None) and self.nproc == 1:
                self.close()
        except Exception:
            pass

    def host_barrier(self):
        if self._side is not None:
            self._dist.barrier(group=self._side)

    @property
    def local_ranks(self):
        return list(range(self.proc * self.L, (self.proc + 1) * self.L))

    # ---- memory -------------------------------------------------------------------------------
    def symm_empty(self, shape, dtype=torch.uint8) -> torch.Tensor:
        """A tensor inside the symmetric heap.  Every process must make the same sequence of
        allocations only if it wants equal offsets; the kernels do not require that."""
        if isinstance(shape, int):
            shape = (shape,)
        numel = int(np.prod(shape)) if len(shape) else 1
        itemsize = torch.empty(0, dtype=dtype).element_size()
        blk = _Block(self, numel * itemsize)
        t = torch.as_tensor(blk, device=f"cuda:{self.device}")
        t = t[: numel * itemsize].view(dtype).view(*shape) if numel else t[:0].view(dtype).view(*shape)
        return t

    def symm_zeros(self, shape, dtype=torch.uint8) -> torch.Tensor:
        t = self.symm_empty(shape, dtype)
        t.zero_()
        return t

    # ---- collectives --------------------------------------------------------------------------
    def _marshal(self, send, recv, sendcounts, sdispls, recvcounts, rdispls, type_size):
        """Normalises the arguments of one collective: pointer arrays, [L, P] count arrays, keep-alive list."""
        L, P = self.L, self.P
        send_l = [send] if isinstance(send, torch.Tensor) else (list(send) if send is not None else [None] * L)
        recv_l = [recv] if isinstance(recv, torch.Tensor) else list(recv)
        if len(send_l) != L or len(recv_l) != L:
            raise ValueError(f"expected {L} send and receive tensors")
        ts = int(type_size) if type_size else recv_l[0].element_size()
        on_dev = isinstance(sendcounts, torch.Tensor) and sendcounts.is_cuda
        keep = [send_l, recv_l]
        if on_dev:
            def dev(a, dt):
                if a is None:
                    return None
                a = a.to(dt).contiguous().view(L, P)
                keep.append(a)
                return a
            sc, rc = dev(sendcounts, torch.int32), dev(recvcounts, torch.int32)
            sd, rd = dev(sdispls, torch.int64), dev(rdispls, torch.int64)
            if sd is None or rd is None:
                raise ValueError("device-resident counts need explicit displacements")
            ptrs = (sc.data_ptr(), rc.data_ptr() if rc is not None else None, sd.data_ptr(), rd.data_ptr())
        else:
            sc = np.ascontiguousarray(np.asarray(sendcounts, dtype=np.int32).reshape(L, P))
            rc = None if recvcounts is None else np.ascontiguousarray(np.asarray(recvcounts, dtype=np.int32).reshape(L, P))
            if sdispls is None:
                sd = np.zeros((L, P), dtype=np.int64)
                sd[:, 1:] = np.cumsum(sc[:, :-1], axis=1)
            else:
                sd = np.ascontiguousarray(np.asarray(sdispls, dtype=np.int64).reshape(L, P))
            if rdispls is None:
                if rc is None:
                    raise ValueError("rdispls or recvcounts is required")
                rd = np.zeros((L, P), dtype=np.int64)
                rd[:, 1:] = np.cumsum(rc[:, :-1], axis=1)
            else:
                rd = np.ascontiguousarray(np.asarray(rdispls, dtype=np.int64).reshape(L, P))
            keep += [sc, rc, sd, rd]
            ptrs = (sc.ctypes.data, rc.ctypes.data if rc is not None else None, sd.ctypes.data, rd.ctypes.data)
        sp = (C.c_void_p * L)(*[(t.data_ptr() if t is not None else None) for t in send_l])
        rp = (C.c_void_p * L)(*[t.data_ptr() for t in recv_l])
        keep += [sp, rp]
        return ts, on_dev, sp, rp, ptrs, keep

    def alltoallv(self, send: Sequence[torch.Tensor] | torch.Tensor, recv: Sequence[torch.Tensor] | torch.Tensor,
                  sendcounts, sdispls=None, recvcounts=None, rdispls=None, *, algo: str = "spreadout",
                  n: int = 0, r: int = 2, r2: int = 0, b: int = 0, b2: int = 0, type_size: Optional[int] = None,
                  inplace: bool = False, grid: int = 0, chunk_bytes: int = 0, bytes_hint: int = -1,
                  eager_max_bytes: int = 0, bulk: Optional[int] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> None:
        """Non-uniform all-to-all of the L local ranks (asynchronous on the current stream).

        ``send`` / ``recv`` are one tensor per local rank (a bare tensor when L == 1); ``recv`` must come
        from :meth:`symm_empty`.  Counts and displacements are in elements, shaped ``[L, P]`` (``[P]`` when
        L == 1): numpy / lists (host) or int32 / int64 CUDA tensors (device-resident, e.g. produced by a
        router kernel).  ``sdispls`` / ``rdispls`` default to the packed layout when counts are on the host.
        ``recvcounts`` is optional: when given, a block larger than its slot is refused (status
        ``truncate``) instead of overrunning the buffer.

        ``eager_max_bytes`` > 0 selects the low-latency eager protocol: blocks (at most that many bytes, the same
        value on every rank) travel as self-validating units into library-owned cells and the receiver copies
        them out, so there is no metadata phase and ``recv`` may be any device memory.  :meth:`max_block_bytes`
        agrees on the value across ranks.
        """
        # Receive buffers outside the symmetric heap cannot be written by peers: the rendezvous protocol then goes
        # through a symmetric bounce buffer (two extra local copies; the eager protocol needs none).
        recv_l = [recv] if isinstance(recv, torch.Tensor) else list(recv)
        bounce = None
        st = stream or torch.cuda.current_stream(self.device)
        if not eager_max_bytes and not inplace:
            outside = [not self._lib.rbv_ctx_in_heap(self._ctx, C.c_void_p(t.data_ptr()), t.numel() * t.element_size())
                       for t in recv_l]
            if any(outside):
                bounce = []
                for t, out in zip(recv_l, outside):
                    if out:
                        bt = self._bounce_for(t)
                        with torch.cuda.stream(st):   # ordered with the collective, whatever the current stream is
                            bt.copy_(t.reshape(-1).view(torch.uint8), non_blocking=True)   # keep what lies between the blocks
                        bounce.append(bt)
                    else:
                        bounce.append(t)
                recv = bounce
                if type_size is None:
                    type_size = recv_l[0].element_size()
        ts, on_dev, sp, rp, (p_sc, p_rc, p_sd, p_rd), keep = self._marshal(
            send, recv, sendcounts, sdispls, recvcounts, rdispls, type_size)
        algo_id = ALGO_ID[algo] if isinstance(algo, str) else int(algo)
        self._lib.rbv_ctx_set_eager(self._ctx, int(eager_max_bytes))
        self._lib.rbv_ctx_set_bulk(self._ctx, int(self._bulk if bulk is None else bulk))
        rcode = self._lib.rbv_alltoallv(self._ctx, algo_id, n, r, r2, b, b2, ts, sp, rp, p_sc, p_rc, p_sd, p_rd,
                                        1 if on_dev else 0, int(bytes_hint), 1 if inplace else 0, int(grid),
                                        int(chunk_bytes), C.c_void_p(st.cuda_stream))
        if rcode:
            raise CommError(f"alltoallv({algo}) failed with code {rcode}: {self._lib.rbv_last_error().decode()}")
        if bounce is not None:
            with torch.cuda.stream(st):
                for t, bt in zip(recv_l, bounce):
                    if bt is not t:
                        t.reshape(-1).view(torch.uint8).copy_(bt, non_blocking=True)

    def _bounce_for(self, t: torch.Tensor) -> torch.Tensor:
        """A symmetric buffer of t's size, kept for reuse (one per size and position in the call)."""
        n = t.numel() * t.element_size()
        cache = self.__dict__.setdefault("_bounce", {})
        key = (n, t.data_ptr())
        if key not in cache:
            cache[key] = self.symm_empty(max(n, 1), torch.uint8)[:n]
        return cache[key]

    def require_same_offsets(self, *offsets: int) -> None:
        """Kernels that address a peer's buffer by its heap offset need that offset to be equal on every rank
        (true when all ranks make the same sequence of equally sized symmetric allocations).  Collective."""
        if self._side is None:
            return
        mine = [int(o) for o in offsets]
        allv = [None] * self.nproc
        self._dist.all_gather_object(allv, mine, group=self._side)
        if any(v != allv[0] for v in allv):
            raise CommError(f"symmetric buffers sit at different heap offsets on different ranks: {allv}")

    def max_block_bytes(self, sendcounts, type_size: int) -> int:
        """Largest block of the whole exchange in bytes (host counts; collective over the processes)."""
        m = int(np.max(np.asarray(sendcounts))) * int(type_size) if np.size(sendcounts) else 0
        if self._side is not None:
            t = torch.tensor([m], dtype=torch.int64)
            self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX, group=self._side)
            m = int(t.item())
        return m

    def prepare(self, send, recv, sendcounts, sdispls=None, recvcounts=None, rdispls=None, *,
                algo: str = "spreadout", n: int = 0, r: int = 2, r2: int = 0, b: int = 0, b2: int = 0,
                type_size: Optional[int] = None, inplace: bool = False, grid: int = 0, chunk_bytes: int = 0,
                bytes_hint: int = -1, eager_max_bytes: int = 0, bulk: Optional[int] = None,
                static: Optional[bool] = None) -> "PreparedCall":
        """Persistent form of :meth:`alltoallv` (compare ``MPI_Alltoallv_init``): everything is resolved once;
        ``.launch()`` then costs one kernel launch.  Buffers and counts are fixed (device-resident counts are
        re-read by every launch, so a router may still change their values).

        With host-side counts the rendezvous protocol is resolved completely on the host: the processes gather
        each other's counts, displacements and buffer offsets over the host side group here, once, and every launch
        runs the static kernel, which has no metadata phase (``static=False`` or ``RBV_STATIC=0`` keeps the
        kernel that exchanges metadata itself).  Collective over the processes.

        ``recv`` tensors outside the symmetric heap (pinned host memory, say) are accepted when the counts are on the
        host (their extents are checked against the tensors here).  When one process hosts every rank the call has no
        peers and addresses everything absolutely: every block goes from the send buffer to the receive buffer in one
        copy.  Otherwise the call receives into symmetric stand-ins and the static kernel copies the received blocks
        on to the tensors itself once everything has arrived, so that the end of the launch is the end of the whole
        transfer (all processes must pass such tensors in the same positions).  ``send`` may be any
        device-accessible memory in every case."""
        ts, on_dev, sp, rp, (p_sc, p_rc, p_sd, p_rd), keep = self._marshal(
            send, recv, sendcounts, sdispls, recvcounts, rdispls, type_size)
        algo_id = ALGO_ID[algo] if isinstance(algo, str) else int(algo)
        if static is None:
            static = os.environ.get("RBV_STATIC", "1") != "0"
        flags = (1 if inplace else 0) | (0 if static else 0x100)
        mirrored, mirror_ptrs = [], None
        if not on_dev and not eager_max_bytes and not inplace and self._recv_extents_fit(recv, keep, ts):
            if self.nproc == 1 and static:
                flags |= 0x200   # receive buffers may be any device-accessible memory; extents checked here
            else:
                # Peers cannot store into memory outside the symmetric heap: the call receives into symmetric
                # stand-ins and the received blocks are copied on to the caller's tensors (by the static kernel
                # itself once everything has arrived, by copies after the launch otherwise).  Collective: every
                # process must pass such tensors in the same positions.
                recv_l = keep[1]
                stand = []
                for t in recv_l:
                    if self._lib.rbv_ctx_in_heap(self._ctx, C.c_void_p(t.data_ptr()), max(t.numel() * t.element_size(), 1)):
                        stand.append(t)
                    else:
                        bt = self._bounce_for(t)
                        stand.append(bt)
                        mirrored.append((t, bt))
                mirror_ptrs = (C.c_void_p * self.L)(*[(t.data_ptr() if bt is not t else None)
                                                      for t, bt in zip(recv_l, stand)])
                ts, on_dev, sp, rp, (p_sc, p_rc, p_sd, p_rd), keep2 = self._marshal(
                    send, stand, sendcounts, sdispls, recvcounts, rdispls, ts)
                keep = keep2 + [keep, mirror_ptrs]
        self._lib.rbv_ctx_set_eager(self._ctx, int(eager_max_bytes))
        self._lib.rbv_ctx_set_bulk(self._ctx, int(self._bulk if bulk is None else bulk))
        g = (None, None, None, None)
        if self.nproc > 1 and not eager_max_bytes and not inplace:
            g = self._gather_global(keep, rp, on_dev or not static)
        self._lib.rbv_ctx_set_recv_mirror(self._ctx, mirror_ptrs)
        h = self._lib.rbv_prepare_global(self._ctx, algo_id, n, r, r2, b, b2, ts, sp, rp, p_sc, p_rc, p_sd, p_rd,
                                         1 if on_dev else 0, int(bytes_hint), flags, int(grid), int(chunk_bytes), *g)
        if not h:
            raise CommError(f"prepare({algo}) failed: {self._lib.rbv_last_error().decode()}")
        return PreparedCall(self, h, keep, mirrored)

    def _recv_extents_fit(self, recv, keep, ts: int) -> bool:
        """True when some receive tensor lies outside the symmetric heap and every block of every rank
        (displacement + count, from the host-side arrays of ``keep``) ends inside its tensor.  Only then may a
        single-process static call be told that its receive buffers can be anywhere."""
        recv_l = [recv] if isinstance(recv, torch.Tensor) else list(recv)
        if all(self._lib.rbv_ctx_in_heap(self._ctx, C.c_void_p(t.data_ptr()), max(t.numel() * t.element_size(), 1))
               for t in recv_l):
            return False
        sc, rc, rd = keep[2], keep[3], keep[5]
        if rd is None or (rc is None and self.L != self.P):
            return False
        cnt = np.asarray(rc if rc is not None else np.asarray(sc).T, dtype=np.int64).reshape(self.L, self.P)
        ext = ((np.asarray(rd, dtype=np.int64).reshape(self.L, self.P) + np.maximum(cnt, 0)) * ts).max(axis=1)
        return all(int(ext[i]) <= t.numel() * t.element_size() for i, t in enumerate(recv_l))

    def _gather_global(self, keep, rp, opt_out: bool):
        """All processes' host-side arguments of one call, as the four tables ``rbv_prepare_global`` takes (or four
        ``None`` when some process cannot take part: device-resident counts, static resolution switched off).
        ``keep`` is the list :meth:`_marshal` built (..., sc, rc, sd, rd, ...), ``rp`` its receive pointers."""
        sc, rc, sd, rd = keep[2:6] if not opt_out else (None, None, None, None)
        mine = None
        if not opt_out:
            base = int(self._lib.rbv_ctx_heap(self._ctx, self.proc))
            off = np.array([int(p) - base for p in rp], dtype=np.uint64)
            mine = (sc, rc, rd, off)
        allv = [None] * self.nproc
        self._dist.all_gather_object(allv, mine, group=self._side)
        if any(v is None for v in allv):
            return (None, None, None, None)
        g_counts = np.ascontiguousarray(np.concatenate([v[0] for v in allv], axis=0), dtype=np.int32)
        have_caps = all(v[1] is not None for v in allv)
        g_caps = np.ascontiguousarray(np.concatenate([v[1] for v in allv], axis=0), dtype=np.int32) if have_caps else None
        g_rd = np.ascontiguousarray(np.concatenate([v[2] for v in allv], axis=0), dtype=np.int64)
        g_off = np.ascontiguousarray(np.concatenate([v[3] for v in allv]), dtype=np.uint64)
        keep += [g_counts, g_caps, g_rd, g_off]
        return (g_counts.ctypes.data, g_caps.ctypes.data if g_caps is not None else None, g_rd.ctypes.data,
                g_off.ctypes.data)

    # ---- status -------------------------------------------------------------------------------
    def trace(self) -> list:
        """Per-key time stamps of the most recent call made with :meth:`enable_trace` on: one entry per key of the
        schedule (a round or a batch), ``{"phase", "step", "start_us", "end_us"}`` relative to the first start;
        phase 0 self copies, 1 intra-group / flat rounds, 2 inter-group, 3 hand-out, 255 eager unpacking."""
        n = 257
        keys, t0, t1 = (C.c_uint * n)(), (C.c_ulonglong * n)(), (C.c_ulonglong * n)()
        self._lib.rbv_ctx_set_stream(self._ctx, C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        m = self._lib.rbv_ctx_last_trace(self._ctx, keys, t0, t1, n)
        rows = [(int(keys[i]), int(t0[i]), int(t1[i])) for i in range(m) if int(t0[i]) != 2 ** 64 - 1 and int(t1[i])]
        if not rows:
            return []
        base = min(r[1] for r in rows)
        return [{"phase": k >> 24, "step": k & 0xffffff, "start_us": (a - base) / 1e3, "end_us": (b - base) / 1e3}
                for k, a, b in rows]

    def status(self) -> dict:
        """Synchronises the current stream and returns the device-side status of the last call."""
        st = Status()
        self._lib.rbv_ctx_set_stream(self._ctx, C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        self._lib.rbv_ctx_status(self._ctx, C.byref(st))
        tr = [int(x) for x in st.trace]
        return {"code": st.code, "name": STATUS_NAMES.get(st.code, "?"), "site": SITE_NAMES.get(st.site, "?"),
                "detail": (st.detail0, st.detail1), "trace_ns": tr,
                "phases_us": {"publish": (tr[1] - tr[0]) / 1e3, "metadata": (tr[2] - tr[1]) / 1e3,
                              "issue": (tr[3] - tr[2]) / 1e3, "drain": (tr[4] - tr[3]) / 1e3,
                              "fence": (tr[6] - tr[5]) / 1e3, "copy": (tr[5] - tr[2]) / 1e3, "report": (tr[7] - tr[6]) / 1e3}}

    def check(self) -> None:
        s = self.status()
        if s["code"]:
            raise CommError(f"device status {s['name']} at {s['site']} detail={s['detail']}")

    def reset(self) -> None:
        """Clears flags and counters after an error.  Collective: every process must call it."""
        torch.cuda.synchronize(self.device)
        self.host_barrier()
        self._lib.rbv_ctx_reset(self._ctx)
        self.host_barrier()

    def set_bulk(self, mode: int) -> None:
        """Bulk-copy engine (``cp.async.bulk`` through a shared-memory ring per warp) for large 16-byte aligned
        chunks of the rendezvous protocol: 0 = never (default; the vector path measured as fast), 1 = whenever the
        buffers allow, -1 = chosen by size."""
        self._bulk = int(mode)
        self._lib.rbv_ctx_set_bulk(self._ctx, self._bulk)

    def enable_trace(self, on: bool = True) -> None:
        """Have every following call report its phase time stamps (``status()['phases_us']``)."""
        self._lib.rbv_ctx_set_trace(self._ctx, 1 if on else 0)

    def set_cooperative(self, mode) -> None:
        """Kernel launch mode: ``None`` / -1 cooperative only where a call needs all its CTAs resident (default),
        ``True`` / 1 always cooperative, ``False`` / 0 never (in-place calls excepted)."""
        m = -1 if mode is None else int(mode)
        self._lib.rbv_ctx_set_cooperative(self._ctx, -1 if m < 0 else (1 if m else 0))

    def set_timeout_ms(self, ms: float) -> None:
        self._lib.rbv_ctx_set_timeout_ms(self._ctx, float(ms))

    # ---- liveness on the host ------------------------------------------------------------------
    # A process that stops taking part (between calls, with nothing of its own in flight) says so in the job's
    # key-value store; the others look before they launch, so that nobody spins on the device for a peer that
    # will not come.  A process that vanishes without a word is caught by the device-side deadline instead.
    def _store(self):
        if self._dist is None:
            return None
        from torch.distributed import distributed_c10d as c10d
        return c10d._get_default_store()

    def announce_leave(self) -> None:
        st = self._store()
        if st is not None:
            st.set(f"rbv/left/{self.proc}", "1")

    def announce_return(self) -> None:
        st = self._store()
        if st is not None:
            st.set(f"rbv/left/{self.proc}", "0")

    def departed(self) -> list:
        """Processes that have announced that they left (and not that they returned)."""
        st = self._store()
        if st is None:
            return []
        out = []
        for q in range(self.nproc):
            key = f"rbv/left/{q}"
            if st.check([key]) and st.get(key) == b"1":
                out.append(q)
        return out

    def require_peers(self) -> None:
        gone = self.departed()
        if gone:
            raise CommError(f"processes {gone} have left the communicator; not launching")

    def inject_absent_rank(self, local_rank: int) -> None:
        """Test hook: the given local rank skips the metadata phase of the following calls (-1 switches it off).
        The other ranks then run into their bounded wait and report a time-out."""
        self._lib.rbv_ctx_set_absent_rank(self._ctx, int(local_rank))

    def plan(self, algo: str, **kw) -> Plan:
        return Plan(algo, self.P, lib=self._lib, **kw)


def init(nranks: Optional[int] = None, **kw) -> Communicator:
    """Creates (or returns) the process-wide default communicator."""
    global _default_comm
    if _default_comm is None or (nranks and _default_comm.P != nranks):
        _default_comm = Communicator(nranks, **kw)
    return _default_comm


def get_default_comm() -> Communicator:
    if _default_comm is None:
        raise CommError("call rbruck_alltoallv_b200.init() first")
    return _default_comm
