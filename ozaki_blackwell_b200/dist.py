"""Row-block sharded FP64 product over the GPUs of one node.

The reference is single-GPU (it has no multi-device code at all); this module adds the one distributed strategy the
product admits without changing a single bit of the result: rank g owns a block of rows of A and produces the same rows
of C. Row scales are local to those rows; column scales and residues of B are recomputed identically on every rank, so
the only exchange is one broadcast of B from the rank that holds it, on a communication stream. Two ways to cut it:

* "rows" (chosen when B is at most 1 GiB): B travels as whole rows, straight out of the source's tensor (no packing),
  and the GEMMs and the reconstruction run once, over the full width. In one piece, the exposed cost is the broadcast
  minus the residues of A that run beside it. In several pieces, the source first reduces the column maxima of its B and
  sends those 8 n bytes ahead, so that every receiver turns each chunk of rows into residues the moment it lands.
* "panels" (chosen for a larger B, in pieces of about 1 GiB): B travels in column panels (whole columns, packed panel-major on the source first), and each panel
  is scaled, multiplied and reconstructed as soon as it lands. More overlap, but narrower GEMM launches and a packing copy.

Measured on two B200s, 16 moduli: at n = 8192 (B = 512 MiB) one row chunk 7.39 ms per product, two panels 7.75, four
panels 7.86, against 7.03 on one GPU without any transfer; the single transfer leaves about 0.35 ms exposed, less than
the panels' narrower launches cost. Row chunks with the maxima sent ahead do not beat the single piece either: 8.02 ms with
two chunks, 7.39 when the communication stream is given high priority (a transfer kernel launched while another kernel's
blocks are still being dispatched otherwise waits for them), which is what one piece takes without it. At n = 32768 (B = 8 GiB) the transfer would leave tens of milliseconds exposed, and
panels hide all but the first.

Peer memory is never read by a kernel of this library: B is in the GPU's own HBM before any kernel touches it.

One process per GPU, `torch.distributed` (NCCL over NVLink/NVSwitch on GPUs; the orchestration itself is backend
agnostic and is exercised with gloo on CPU ranks in the tests, with a checker-backed engine injected there).
"""
import ctypes

import torch
import torch.distributed as dist

PANEL_ALIGN = 256   # ozb_plan_panel wants panel starts on multiples of 256 columns (the GEMM's tile width)


def row_block(m_total, rank, world):
    """Rows [lo, hi) of rank `rank`: blocks differ by at most one row, earlier ranks get the longer ones."""
    base, extra = divmod(m_total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


AUTO_PIECE_BYTES = 1 << 30


def choose_layout(k, n, layout="auto", pieces=None):
    """The broadcast layout and the number of pieces for a k x n FP64 B: what was asked for, else by the size of B.
    pieces = 0 with layout "panels" means growing panels (see growing_panels)."""
    nbytes = 8 * k * n
    if layout == "auto":
        layout = "rows" if nbytes <= AUTO_PIECE_BYTES else "panels"
    if pieces is None:
        pieces = 1 if layout == "rows" else 0
    return layout, pieces


def growing_panels(n):
    """Column panels of n/16, 3n/16, n/4 and n/2 columns (starts on multiples of PANEL_ALIGN). The transfer of a panel
    takes about a third of the time its product takes, so the first panel is small (its transfer hides behind the
    residues of A, which need nothing of B), every later one has arrived before the one before it is used up, and most
    of the columns sit in wide panels, whose GEMM launches run best."""
    unit = max(PANEL_ALIGN, (n // 16) // PANEL_ALIGN * PANEL_ALIGN)
    out, start = [], 0
    for width in (unit, 3 * unit, 4 * unit):
        if n - start <= width:
            break
        out.append((start, start + width))
        start += width
    out.append((start, n))
    return out


ROW_ALIGN = 128   # ozb_plan_b_rows_residues wants chunk starts on multiples of 128 rows


def row_chunks(k, chunks):
    """Split k rows into at most `chunks` contiguous ranges of near-equal length whose starts are multiples of ROW_ALIGN."""
    blocks = (k + ROW_ALIGN - 1) // ROW_ALIGN
    chunks = max(1, min(chunks, blocks))
    out, start = [], 0
    for c in range(chunks):
        nb = blocks // chunks + (1 if c < blocks % chunks else 0)
        stop = min(k, start + nb * ROW_ALIGN)
        out.append((start, stop))
        start = stop
    return out


def panel_ranges(n, panels):
    """Split n columns into at most `panels` ranges whose starts are multiples of PANEL_ALIGN."""
    if panels <= 1 or n <= PANEL_ALIGN:
        return [(0, n)]
    blocks = (n + PANEL_ALIGN - 1) // PANEL_ALIGN
    panels = min(panels, blocks)
    out, start = [], 0
    for p in range(panels):
        nb = blocks // panels + (1 if p < blocks % panels else 0)
        stop = min(n, start + nb * PANEL_ALIGN)
        out.append((start, stop))
        start = stop
    return out


class CudaEngine:
    """The product path: a plan of libozaki_blackwell.so on the current CUDA device."""

    def __init__(self, m, n, k, moduli):
        from ._lib import lib
        self._lib = lib
        self._plan = ctypes.c_void_p()
        self._check(lib.ozb_plan_create(m, n, k, moduli, 62, ctypes.byref(self._plan)))
        self.m, self.n, self.k = m, n, k

    def _check(self, code):
        if code:
            raise RuntimeError(self._lib.ozb_error(code).decode())

    @staticmethod
    def _row_major(*tensors):
        for t in tensors:
            if t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.float64:
                raise ValueError("operands must be two-dimensional float64 tensors with unit column stride")

    def set_a(self, a, stream):
        self._row_major(a)
        self._check(self._lib.ozb_plan_set_a(self._plan, a.data_ptr(), a.stride(0), stream.cuda_stream))

    def panel(self, b_panel, c, j0, ncols, stream):
        self._row_major(b_panel, c)
        c_ptr = c.data_ptr() + 8 * j0
        self._check(self._lib.ozb_plan_panel(self._plan, b_panel.data_ptr(), b_panel.stride(0), c_ptr, c.stride(0), j0, ncols,
                                             stream.cuda_stream))

    def b_begin(self, stream):
        self._check(self._lib.ozb_plan_b_begin(self._plan, stream.cuda_stream))

    def b_rows(self, rows, stream):
        self._check(self._lib.ozb_plan_b_rows(self._plan, rows.data_ptr(), rows.stride(0), rows.shape[0], stream.cuda_stream))

    def cols_absmax(self, b, colmax, stream):
        self._check(self._lib.ozb_cols_absmax(b.data_ptr(), b.shape[0], b.shape[1], b.stride(0), colmax.data_ptr(), stream.cuda_stream))

    def b_rows_residues(self, rows, k0, colmax, stream):
        self._check(self._lib.ozb_plan_b_rows_residues(self._plan, rows.data_ptr(), rows.stride(0), k0, rows.shape[0], colmax.data_ptr(),
                                                       stream.cuda_stream))

    def b_finish(self, b, stream):
        self._check(self._lib.ozb_plan_b_finish(self._plan, b.data_ptr(), b.stride(0), stream.cuda_stream))

    def multiply(self, c, stream):
        self._row_major(c)
        self._check(self._lib.ozb_plan_multiply(self._plan, c.data_ptr(), c.stride(0), stream.cuda_stream))

    def full(self, a, b, c, stream):
        self._row_major(a, b, c)
        self._check(self._lib.ozb_plan_dgemm(self._plan, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), c.data_ptr(),
                                             c.stride(0), stream.cuda_stream))

    def status(self):
        self._check(self._lib.ozb_plan_status(self._plan))

    def close(self):
        if self._plan:
            self._lib.ozb_plan_destroy(self._plan)
            self._plan = ctypes.c_void_p()


class NativeSharded:
    """The same product through the library's own multi-GPU layer (ozb_mg_*: NCCL driven from C++, non-blocking
    communicator, bounded host waits). One handle per rank; the rendezvous id travels over the process group."""

    def __init__(self, moduli, group=None, src=0, timeout_ms=0):
        from ._lib import lib
        self._lib, self.moduli, self.src, self.kernels = lib, moduli, src, 0
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            self._check(lib.ozb_mg_unique_id(ident))
        box = [ident.raw]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self._handle = ctypes.c_void_p()
        self._check(lib.ozb_mg_create(world, rank, box[0], timeout_ms, ctypes.byref(self._handle)))

    def _check(self, code):
        if code:
            raise RuntimeError(self._lib.ozb_error(code).decode())

    def __call__(self, a_local, b, c_local, stream, on_host=False):
        m, k = a_local.shape
        n = c_local.shape[1]
        b_ptr, ldb = (b.data_ptr(), b.stride(0)) if b is not None else (None, n)
        self._check(self._lib.ozb_mg_dgemm(self._handle, m, n, k, a_local.data_ptr(), a_local.stride(0), b_ptr, ldb, c_local.data_ptr(),
                                           c_local.stride(0), self.moduli, self.src, 1 if on_host else 0,
                                           None if on_host else stream.cuda_stream))

    def status(self):
        self._check(self._lib.ozb_mg_wait(self._handle))

    def info(self):
        layout, pieces, kernels = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self._check(self._lib.ozb_mg_info(self._handle, ctypes.byref(layout), ctypes.byref(pieces), ctypes.byref(kernels)))
        self.kernels = kernels.value
        return ("whole", "stream")[layout.value], pieces.value

    def close(self):
        if self._handle:
            self._lib.ozb_mg_destroy(self._handle)
            self._handle = ctypes.c_void_p()


class _HostStreams:
    """Stand-ins for CUDA streams and events on CPU ranks (gloo tests): everything is synchronous there."""

    class _S:
        cuda_stream = 0

        def wait_event(self, e):
            pass

        def wait_stream(self, s):
            pass

    class _E:
        def record(self, s=None):
            pass

    def stream(self):
        return self._S()

    def event(self):
        return self._E()


class RowShardedGemm:
    """C_local = A_local @ B with B held by rank `src`; bit-identical to the single-GPU product of the stacked rows.

    m_local, n, k: this rank's block of rows, the width of B/C and the inner length. `engine` defaults to the CUDA
    plan; tests on CPU ranks inject one with the same methods. `panels` is the number of pieces B is broadcast in
    (row chunks for layout "rows", column panels for layout "panels"); both default to a choice by the size of B.
    """

    def __init__(self, m_local, n, k, moduli=16, group=None, src=0, panels=None, engine=None, device=None, layout="auto",
                 native=None, timeout_ms=0):
        if layout not in ("auto", "rows", "panels"):
            raise ValueError("layout is 'auto', 'rows' or 'panels'")
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.n, self.k, self.moduli = m_local, n, k, moduli
        # On GPUs the exchange is driven by the library itself unless a layout of this module is asked for by name; the
        # orchestration below is the same strategy written against torch.distributed (any backend; gloo in the CPU tests).
        if native is None:
            native = engine is None and self.world > 1 and layout == "auto" and panels is None
        self.native = NativeSharded(moduli, group, src, timeout_ms) if native else None
        if self.native:
            self.group, self.src, self.layout, self.ranges = group, src, "native", [(0, k)]
            self.engine, self.compute, self.stage = self.native, torch.cuda.current_stream(), None
            return
        layout, panels = choose_layout(k, n, layout, panels)
        self.group, self.src, self.layout = group, src, layout
        pieces = panels if self.world > 1 else 1
        if layout == "rows":
            self.ranges = row_chunks(k, pieces)
        else:
            self.ranges = growing_panels(n) if pieces == 0 and self.world > 1 else panel_ranges(n, max(1, pieces))
        self.engine = engine if engine is not None else CudaEngine(m_local, n, k, moduli)
        self.on_gpu = engine is None or (device is not None and torch.device(device).type == "cuda")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if self.on_gpu:
            self.compute = torch.cuda.current_stream()
            self.comm = torch.cuda.Stream()
            self.pack = torch.cuda.Stream()
            self._event = lambda: torch.cuda.Event()
        else:
            hs = _HostStreams()
            self.compute, self.comm, self.pack, self._event = hs.stream(), hs.stream(), hs.stream(), hs.event
        if self.world == 1:
            self.stage = None
        elif layout == "panels":   # panel-major staging: panel p is a contiguous k x width block, broadcast as one buffer
            self.stage = [torch.empty((k, hi - lo), dtype=torch.float64, device=self.device) for lo, hi in self.ranges]
        else:                      # the receivers' copy of B (the source sends from its own tensor when that is contiguous)
            self.stage = torch.empty((k, n), dtype=torch.float64, device=self.device)
            self.colmax = torch.zeros(n, dtype=torch.int64, device=self.device)   # bit patterns of the column maxima of |B|

    def __call__(self, a_local, b, c_local):
        """a_local [m_local, k], c_local [m_local, n]; b [k, n] is read on rank `src` only (others may pass None)."""
        if self.native:
            if self.rank == self.src and b.stride(1) != 1:
                b = b.contiguous()
            self.native(a_local, b if self.rank == self.src else None, c_local, torch.cuda.current_stream())
            if self.layout == "native":
                self.layout, pieces = self.native.info()
                self.ranges = [(0, self.k)] * pieces
            return c_local
        if self.world == 1:
            self.engine.full(a_local, b, c_local, self.compute)
            return c_local
        if self.rank == self.src and b.stride(1) != 1:
            b = b.contiguous()                      # the kernels take a row pitch, not a column stride
        if self.layout == "rows":
            return self._by_rows(a_local, b, c_local)
        # The source packs each panel (panel-major, contiguous) on a stream of its own, broadcasts it as soon as it is
        # packed, and computes from its own B directly: its compute stream waits for nothing.
        src = self.rank == self.src
        start = self._event()
        start.record(self.compute)                 # orders this call after the caller's writes of A and B
        ctx = (lambda s: torch.cuda.stream(s)) if self.on_gpu else (lambda s: _null())
        packed = []
        if src:
            self.pack.wait_event(start)
            with ctx(self.pack):
                for (lo, hi), buf in zip(self.ranges, self.stage):
                    buf.copy_(b[:, lo:hi])
                    ev = self._event()
                    ev.record(self.pack)
                    packed.append(ev)
        arrived = []
        with ctx(self.comm):
            for p, buf in enumerate(self.stage):
                if src:
                    self.comm.wait_event(packed[p])
                dist.broadcast(buf, src=self.src, group=self.group)
                ev = self._event()
                ev.record(self.comm)
                arrived.append(ev)
        self.engine.set_a(a_local, self.compute)   # overlaps the first panel's transfer
        for (lo, hi), buf, ev in zip(self.ranges, self.stage, arrived):
            if src:
                self.engine.panel(b[:, lo:hi], c_local, lo, hi - lo, self.compute)
            else:
                self.compute.wait_event(ev)
                self.engine.panel(buf, c_local, lo, hi - lo, self.compute)
        # the staging buffers may be overwritten by the next call only after this one's reads
        self.comm.wait_stream(self.compute)
        if src:
            self.pack.wait_stream(self.comm)
            self.compute.wait_stream(self.pack)    # the caller may overwrite B on the compute stream after this call
        return c_local

    def _by_rows(self, a_local, b, c_local):
        if len(self.ranges) > 1:
            return self._by_rows_maxima_first(a_local, b, c_local)
        if self.rank == self.src and b.is_contiguous():
            whole = b                               # sent in place, nothing staged
        else:
            whole = self.stage
            if self.rank == self.src:
                whole.copy_(b)
        ready = self._event()
        ready.record(self.compute)                  # orders the copy above, and the previous call's reads of the stage
        self.comm.wait_event(ready)
        ctx = torch.cuda.stream(self.comm) if self.on_gpu else _null()
        with ctx:
            dist.broadcast(whole, src=self.src, group=self.group)
            arrived = self._event()
            arrived.record(self.comm)
        self.engine.b_begin(self.compute)
        self.engine.set_a(a_local, self.compute)    # beside the transfer
        if whole is self.stage:                     # a receiver, or a source that staged a strided B
            self.compute.wait_event(arrived)
        self.engine.b_rows(whole, self.compute)
        self.engine.b_finish(whole, self.compute)
        self.engine.multiply(c_local, self.compute)
        self.comm.wait_stream(self.compute)
        if whole is b:
            self.compute.wait_stream(self.comm)     # B was sent in place: the caller may overwrite it only after the sends
        return c_local

    def _by_rows_maxima_first(self, a_local, b, c_local):
        """Several row chunks: the source first reduces the column maxima of its B (one pass) and sends those 8 n bytes
        ahead, so that every receiver can turn each chunk of rows into residues the moment it lands."""
        src = self.rank == self.src
        in_place = src and b.is_contiguous()
        whole = b if in_place else self.stage
        if src:
            if not in_place:
                whole.copy_(b)
            self.colmax.zero_()
            self.engine.cols_absmax(whole, self.colmax, self.compute)
        ready = self._event()
        ready.record(self.compute)
        self.comm.wait_event(ready)
        arrived = []
        ctx = torch.cuda.stream(self.comm) if self.on_gpu else _null()
        with ctx:
            dist.broadcast(self.colmax, src=self.src, group=self.group)
            for lo, hi in self.ranges:
                dist.broadcast(whole[lo:hi], src=self.src, group=self.group)
                ev = self._event()
                ev.record(self.comm)
                arrived.append(ev)
        self.engine.set_a(a_local, self.compute)    # beside the transfer
        if src:
            self.engine.b_rows_residues(whole, 0, self.colmax, self.compute)
        else:
            for (lo, hi), ev in zip(self.ranges, arrived):
                self.compute.wait_event(ev)         # the maxima were sent before the first chunk on the same stream
                self.engine.b_rows_residues(whole[lo:hi], lo, self.colmax, self.compute)
        self.engine.multiply(c_local, self.compute)
        self.comm.wait_stream(self.compute)
        if in_place:
            self.compute.wait_stream(self.comm)
        return c_local

    def host(self, a_host, b_host, c_host):
        """The product on host operands (pinned memory), copies pipelined with the broadcast and the computation inside the
        library; synchronous. Native path only."""
        if not self.native:
            raise RuntimeError("host operands go through the library's own multi-GPU layer")
        self.native(a_host, b_host if self.rank == self.src else None, c_host, None, on_host=True)
        return c_host

    def close(self):
        close = getattr(self.engine, "close", None)
        if close:
            close()


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
