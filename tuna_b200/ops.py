"""Host-side mirror of the reference's two ops (extension.cpp:26-49).

The reference performs no checks at all (no dtype, device, contiguity or shape
validation, extension.cpp:26-49; unknown shapes silently do nothing,
kernel.cu:3022-3155).  The mirror keeps the call signature and adds the checks:
a bad argument raises instead of corrupting memory.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import TunaConfig, check

_workspaces: dict = {}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _expect(t: torch.Tensor, name: str, dtype, numel: int, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if t.numel() != numel:
        raise ValueError(f"{name} has {t.numel()} elements, expected {numel}")


def workspace_for(m: int, n: int, k: int, device) -> torch.Tensor:
    """A zero-initialised per-(device, stream) workspace large enough for (m, n, k).

    The kernels leave the workspace clean after every call, so one buffer serves
    consecutive calls on a stream; it only grows.
    """
    lib = _lib.load()
    with torch.cuda.device(device):
        need = int(lib.tuna_matmul_workspace_bytes(m, n, k))
    key = (torch.device(device).index, _stream_ptr(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def lookup_config(m: int, n: int, k: int) -> TunaConfig:
    cfg = TunaConfig()
    check(_lib.load().tuna_lookup_config(m, n, k, ctypes.byref(cfg)))
    return cfg


def matmul(x, q, s, c, o, m: int, n: int, k: int, *, config: TunaConfig | None = None, workspace=None) -> None:
    """`tuna.matmul(x, q, s, c, o, m, n, k)` (extension.cpp:26-38).

    x fp16 [n,k]; q uint8 [m/8,k/8,32]; s fp32 [m] (absmax); c fp32 [16]
    (codebook); o fp16 [n,m], overwritten.  Enqueued on the current stream of
    x's device.
    """
    dev = x.device if isinstance(x, torch.Tensor) else None
    _expect(x, "x", torch.float16, n * k)
    _expect(q, "q", torch.uint8, m * k // 2, dev)
    _expect(s, "s", torch.float32, m, dev)
    _expect(c, "c", torch.float32, 16, dev)
    _expect(o, "o", torch.float16, n * m, dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = workspace if workspace is not None else workspace_for(m, n, k, dev)
        args = (q.data_ptr(), x.data_ptr(), c.data_ptr(), s.data_ptr(), o.data_ptr(), m, n, k,
                ws.data_ptr(), ws.numel() * ws.element_size(), _stream_ptr(dev))
        if config is None:
            check(lib.tuna_matmul(*args))
        else:
            check(lib.tuna_matmul_cfg(*args, ctypes.byref(config)))


def matmul_batched(x, q, s, c, o, m: int, n: int, k: int, *, workspace=None) -> None:
    """`batch` independent GEMMs of one shape in one call (one launch for n <= 32):
    `q` uint8 `[batch, m/8, k/8, 32]`, `s` fp32 `[batch, m]`, `o` fp16 `[batch, n, m]`, and `x` fp16
    either `[batch, n, k]` (per-matrix activations, e.g. one token list per expert) or `[n, k]`
    (shared: the reference's "combined" Mixtral GEMM, make_configs.py:105-106)."""
    if not isinstance(q, torch.Tensor) or q.dim() != 4:
        raise ValueError("q must be a [batch, m/8, k/8, 32] tensor")
    batch = q.shape[0]
    dev = q.device
    _expect(q, "q", torch.uint8, batch * m * k // 2, dev)
    _expect(s, "s", torch.float32, batch * m, dev)
    _expect(c, "c", torch.float32, 16, dev)
    _expect(o, "o", torch.float16, batch * n * m, dev)
    shared = x.dim() == 2
    _expect(x, "x", torch.float16, n * k if shared else batch * n * k, dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        need = int(lib.tuna_matmul_batched_workspace_bytes(m, n, k, batch))
        if workspace is None:
            key = ("batched", dev.index, torch.cuda.current_stream(dev).cuda_stream)
            ws = _workspaces.get(key)
            if ws is None or ws.numel() < need:
                ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
                _workspaces[key] = ws
        else:
            ws = workspace
        check(lib.tuna_matmul_batched(q.data_ptr(), x.data_ptr(), c.data_ptr(), s.data_ptr(), o.data_ptr(), m, n, k, batch,
                                      m * k // 2, 0 if shared else n * k * 2, m * 4, n * m * 2,
                                      ws.data_ptr(), ws.numel(), _stream_ptr(dev)))


class MatmulSequence:
    """`count` independent GEMMs issued as ONE persistent launch (`tuna_matmul_sequence`).

    Built once from the tensors of every GEMM - `gemms` is a list of `(x, q, s, o, m, n, k)` with the
    layouts of `matmul`, `c` the shared codebook - and run any number of times with `run()`, on the
    current stream of the tensors' device.  The tensors are referenced, not copied: their
    contents may change between runs, their addresses may not.  The inputs of all the GEMMs must
    be ready when `run()` is enqueued (the GEMMs do not depend on each other)."""

    def __init__(self, gemms, c, *, workspace=None):
        if not gemms:
            raise ValueError("an empty sequence")
        self.device = gemms[0][0].device
        self.count = len(gemms)
        self._keep = []
        self._descs = (_lib.TunaGemmDesc * self.count)()
        for i, (x, q, s, o, m, n, k) in enumerate(gemms):
            if n == 0:  # an expert without tokens: the entry is skipped by the library
                self._descs[i] = _lib.TunaGemmDesc(q.data_ptr(), 0, s.data_ptr(), 0, m, 0, k, 0)
                self._keep.append((q, s))
                continue
            _expect(x, "x", torch.float16, n * k, self.device)
            _expect(q, "q", torch.uint8, m * k // 2, self.device)
            _expect(s, "s", torch.float32, m, self.device)
            _expect(o, "o", torch.float16, n * m, self.device)
            self._descs[i] = _lib.TunaGemmDesc(q.data_ptr(), x.data_ptr(), s.data_ptr(), o.data_ptr(), m, n, k, 0)
            self._keep.append((x, q, s, o))
        _expect(c, "c", torch.float32, 16, self.device)
        self.code = c
        lib = _lib.load()
        with torch.cuda.device(self.device):
            need = int(lib.tuna_matmul_sequence_workspace_bytes(self._descs, self.count))
            if need == 0:
                raise ValueError("a GEMM of the sequence has an unsupported shape (m and k multiples of 8, n >= 1)")
            if workspace is None:
                workspace = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=self.device)
            elif workspace.numel() * workspace.element_size() < need:
                raise ValueError("workspace too small for this sequence")
        self.workspace = workspace

    def run(self) -> None:
        with torch.cuda.device(self.device):
            check(_lib.load().tuna_matmul_sequence(self._descs, self.count, self.code.data_ptr(), self.workspace.data_ptr(),
                                                   self.workspace.numel() * self.workspace.element_size(), _stream_ptr(self.device)))


class Exchange:
    """The exchange buffers of a tensor-parallel group for `ReduceSequence` (`tuna_exchange`).

    Every rank allocates one buffer of `nbytes` through the library (`tuna_exchange_create`), the
    64-byte IPC handles travel through `torch.distributed` (`all_gather_object` on `group`, any
    backend) and every rank maps its peers' buffers (`tuna_exchange_open`).  With `group=None` the
    exchange has one rank (the sum of one slab): the same code path on a single GPU."""

    def __init__(self, nbytes: int, device, group=None):
        import ctypes

        self.device = torch.device(device)
        lib = _lib.load()
        self._lib = lib
        self.nbytes = int(nbytes)
        self._local = ctypes.c_void_p()
        self._peers = {}
        self._group = group
        self._barrier_on_close = False  # set once every rank is known to hold a working exchange
        self.rank, self.world = 0, 1
        dist = None
        if group is not None:
            import torch.distributed as dist

            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
            if self.world > _lib.MAX_PEERS:
                raise ValueError(f"at most {_lib.MAX_PEERS} ranks")
        # A rank that fails still takes part in both collectives, so that all ranks raise together.
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        try:
            with torch.cuda.device(self.device):
                status = lib.tuna_exchange_create(self.nbytes, ctypes.byref(self._local), handle)
        except Exception:  # no usable CUDA device in this process
            status = -7
        mine = handle.raw if status == 0 else None
        handles = [mine]
        if dist is not None:
            handles = [None] * self.world
            dist.all_gather_object(handles, mine, group=group)
        if any(h is None for h in handles):
            self.close()
            raise RuntimeError("exchange: a rank could not allocate or export its buffer" + (f" (this rank: status {status})" if status else ""))
        self.struct = _lib.TunaExchange()
        self.struct.rank, self.struct.world, self.struct.bytes = self.rank, self.world, self.nbytes
        status = 0
        with torch.cuda.device(self.device):
            for j in range(self.world):
                if j == self.rank:
                    self.struct.buffer[j] = self._local.value
                    continue
                ptr = ctypes.c_void_p()
                status = lib.tuna_exchange_open(handles[j], ctypes.byref(ptr))
                if status != 0:
                    break
                self._peers[j] = ptr
                self.struct.buffer[j] = ptr.value
        oks = [status == 0]
        if dist is not None:
            oks = [None] * self.world
            dist.all_gather_object(oks, status == 0, group=group)  # also: nobody launches before every mapping exists
        if not all(oks):
            self._barrier_on_close = True  # every rank takes this branch: unmap, meet, free
            self.close()
            raise RuntimeError("exchange: a rank could not map a peer's buffer" + (f" (this rank: status {status})" if status else ""))
        self._barrier_on_close = True

    def close(self) -> None:
        """Unmaps the peers' buffers, waits for the other ranks to have done the same (a barrier on
        the group: an exported buffer must outlive its mappings), then frees this rank's buffer.
        Call it on every rank, with no launch on the exchange in flight."""
        have_local = self._local is not None and bool(self._local.value)
        if self._peers or have_local:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                for ptr in self._peers.values():
                    self._lib.tuna_exchange_close(ptr)
        self._peers = {}
        if self._group is not None and self._barrier_on_close:
            import torch.distributed as dist

            dist.barrier(group=self._group)
        if have_local:
            with torch.cuda.device(self.device):
                self._lib.tuna_exchange_destroy(self._local)
        self._local = None


class ReduceSequence(MatmulSequence):
    """K-split GEMMs of a tensor-parallel group in one persistent launch, their partial outputs
    summed over the ranks by the library (`tuna_matmul_sequence_reduce`) instead of a collective:
    after `run()` every rank's `o` tensors hold the sum over ranks (added in rank order in fp32).
    `gemms` as for `MatmulSequence` with this rank's K slice of q and x; every rank passes the same
    shapes and token counts (1..64) in the same order.  `partial` (one bool per GEMM, default all
    True) marks the K-split GEMMs; the others are ordinary GEMMs that share the launch (the
    column-parallel GEMMs of the same layers).  `exchange` is an `Exchange` of at least
    `ReduceSequence.exchange_bytes(shapes, world)` bytes."""

    @staticmethod
    def exchange_bytes(shapes, world: int, partial=None) -> int:
        """Bytes every rank's exchange buffer needs for GEMMs of `shapes` = [(m, n, k), ...]."""
        descs = (_lib.TunaGemmDesc * len(shapes))()
        for i, (m, n, k) in enumerate(shapes):
            descs[i] = _lib.TunaGemmDesc(0, 0, 0, 0, m, n, k, _lib.GEMM_PARTIAL if partial is None or partial[i] else 0)
        return int(_lib.load().tuna_exchange_bytes(descs, len(shapes), world))

    def __init__(self, gemms, c, exchange: Exchange, *, partial=None, workspace=None):
        if any(g[5] < 1 or g[5] > 64 for g in gemms):
            raise ValueError("token counts of a reduce sequence must be 1..64")
        super().__init__(gemms, c, workspace=workspace)
        for i in range(self.count):
            self._descs[i].flags = _lib.GEMM_PARTIAL if partial is None or partial[i] else 0
        self.exchange = exchange
        need = self.exchange_bytes([(g[4], g[5], g[6]) for g in gemms], exchange.world, partial)
        if exchange.nbytes < need:
            raise ValueError(f"exchange buffers too small: {exchange.nbytes} < {need}")

    def run(self) -> None:
        import ctypes

        with torch.cuda.device(self.device):
            check(_lib.load().tuna_matmul_sequence_reduce(self._descs, self.count, self.code.data_ptr(), self.workspace.data_ptr(),
                                                          self.workspace.numel() * self.workspace.element_size(),
                                                          ctypes.byref(self.exchange.struct), _stream_ptr(self.device)))


def _byte_span(first: torch.Tensor, nbytes: int) -> torch.Tensor:
    """A uint8 view of `nbytes` bytes of `first`'s storage, starting where `first` starts."""
    storage = first.untyped_storage()
    offset = first.storage_offset() * first.element_size()
    return torch.empty(0, dtype=torch.uint8, device=first.device).set_(storage, offset, (nbytes,))


def _merge_copies(copies):
    """[(dst, src), ...] contiguous tensors -> the same bytes as fewer, larger copies: runs whose
    destinations follow one another in memory and whose sources do too (same storages) become one."""
    runs = []
    for dst, src in copies:
        nbytes = dst.numel() * dst.element_size()
        if runs:
            d0, s0, n0 = runs[-1]
            same = (d0.untyped_storage().data_ptr() == dst.untyped_storage().data_ptr()
                    and s0.untyped_storage().data_ptr() == src.untyped_storage().data_ptr())
            if same and d0.data_ptr() + n0 == dst.data_ptr() and s0.data_ptr() + n0 == src.data_ptr():
                runs[-1] = (d0, s0, n0 + nbytes)
                continue
        runs.append((dst, src, nbytes))
    return [(dst, src) if n == dst.numel() * dst.element_size() else (_byte_span(dst, n), _byte_span(src, n)) for dst, src, n in runs]


class HostSequence:
    """`MatmulSequence` for callers whose activations and outputs live in (pinned) HOST memory.

    The sequence is cut into `groups` contiguous groups; group j's activations are copied to the
    device on a copy-in stream while group j-1 runs (one persistent launch per group, on the
    caller's current stream) and group j-2's outputs travel back on a copy-out stream.
    `gemms` is a list of `(x_host, q, s, o_host, m, n, k)`: pinned host tensors for x and o, device
    tensors for the weights and scales (they are parameters and stay resident, as in the
    reference).  `run()` returns at once; the current stream has waited for every copy-out when
    it returns, so a stream or event synchronisation after it makes the host outputs readable.
    `after_group(pools)` (optional) runs on the compute stream between a group's launch and its
    copy-out; `pools` maps a pool id to ONE contiguous device tensor holding the outputs of the
    group's GEMMs with that id (`pool_ids`, one int per GEMM, default 0) - e.g. the K-split layers'
    partial outputs, which one all-reduce then sums.  Host tensors that follow one another in one
    pinned allocation travel as one copy per group and pool.  With `exchange` (an `Exchange`) the groups
    run as `ReduceSequence`s: the GEMMs marked in `partial` (default all) are K slices whose outputs
    come back summed over the ranks, without a collective.  A `run()` can be captured into a CUDA graph
    (the host buffers are then fixed addresses read and written at every replay)."""

    def __init__(self, gemms, c, *, groups: int = 4, after_group=None, pool_ids=None, exchange=None, partial=None):
        if not gemms:
            raise ValueError("an empty sequence")
        self.device = gemms[0][1].device
        self.after_group = after_group
        partial = list(partial) if partial is not None else None
        self.copy_in = torch.cuda.Stream(device=self.device)
        self.copy_out = torch.cuda.Stream(device=self.device)
        groups = max(1, min(int(groups), len(gemms)))
        bounds = [round(i * len(gemms) / groups) for i in range(groups + 1)]
        self._groups = []
        workspace = None
        pool_ids = list(pool_ids) if pool_ids is not None else [0] * len(gemms)
        for j in range(groups):
            part = gemms[bounds[j]:bounds[j + 1]]
            ids = pool_ids[bounds[j]:bounds[j + 1]]
            # one slab per pool: the outputs of a pool's GEMMs lie back to back (16-byte aligned pieces)
            sizes = {}
            for (xh, q, s_, oh, m, n, k), pid in zip(part, ids):
                sizes[pid] = sizes.get(pid, 0) + (n * m + 7) // 8 * 8
            slabs = {pid: torch.empty(sz, dtype=torch.float16, device=self.device) for pid, sz in sizes.items()}
            used = {pid: 0 for pid in sizes}
            # the group's activations also lie back to back on the device (16-byte aligned pieces)
            x_slab = torch.empty(sum((n * k + 7) // 8 * 8 for (_xh, _q, _s, _oh, _m, n, k) in part), dtype=torch.float16, device=self.device)
            x_used = 0
            dev_gemms, pairs = [], []
            for (xh, q, s_, oh, m, n, k), pid in zip(part, ids):
                if not (xh.is_pinned() and oh.is_pinned()):
                    raise ValueError("HostSequence needs pinned host tensors (pageable copies would serialise)")
                xd = x_slab[x_used:x_used + n * k].view(n, k)
                x_used += (n * k + 7) // 8 * 8
                od = slabs[pid][used[pid]:used[pid] + n * m].view(n, m)
                used[pid] += (n * m + 7) // 8 * 8
                dev_gemms.append((xd, q, s_, od, m, n, k))
                pairs.append((xh, xd, oh, od))
            # every group sizes its own workspace; the largest one then serves all (one stream, one after the other)
            if exchange is not None:  # the K-split GEMMs of the group are summed over the ranks inside the launch
                seq = ReduceSequence(dev_gemms, c, exchange, partial=partial[bounds[j]:bounds[j + 1]] if partial is not None else None)
            else:
                seq = MatmulSequence(dev_gemms, c)
            if workspace is None or seq.workspace.numel() > workspace.numel():
                workspace = seq.workspace
            # copies of neighbouring tensors (adjacent in host memory AND on the device) are issued as one
            by_pool = sorted(range(len(pairs)), key=lambda i: (ids[i], i))
            self._groups.append({"seq": seq, "pairs": pairs, "pools": slabs, "in": torch.cuda.Event(), "done": torch.cuda.Event(), "out": torch.cuda.Event(),
                                 "copies_in": _merge_copies([(pairs[i][1], pairs[i][0]) for i in range(len(pairs))]),
                                 "copies_out": _merge_copies([(pairs[i][2], pairs[i][3]) for i in by_pool])})
        for g in self._groups:
            g["seq"].workspace = workspace
        self._fork = torch.cuda.Event()
        self.copy_in.wait_stream(torch.cuda.current_stream(self.device))
        self.copy_out.wait_stream(torch.cuda.current_stream(self.device))

    def run(self) -> None:
        compute = torch.cuda.current_stream(self.device)
        # everything enqueued so far (the previous run's launches included) precedes this run's copies
        self._fork.record(compute)
        self.copy_in.wait_event(self._fork)
        self.copy_out.wait_event(self._fork)
        for g in self._groups:
            with torch.cuda.stream(self.copy_in):
                for dst, src in g["copies_in"]:
                    dst.copy_(src, non_blocking=True)
                g["in"].record(self.copy_in)
            compute.wait_event(g["in"])
            g["seq"].run()
            if self.after_group is not None:
                self.after_group(g["pools"])
            g["done"].record(compute)
            self.copy_out.wait_event(g["done"])
            with torch.cuda.stream(self.copy_out):
                for dst, src in g["copies_out"]:
                    dst.copy_(src, non_blocking=True)
                g["out"].record(self.copy_out)
        for g in self._groups:
            compute.wait_event(g["out"])


def matmul_sequence(gemms, c, *, workspace=None) -> None:
    """One-shot form of `MatmulSequence`: `gemms` is a list of `(x, q, s, o, m, n, k)`."""
    MatmulSequence(gemms, c, workspace=workspace).run()


def dequant(q, absmax, codebook, o, m: int, k: int) -> None:
    """`tuna.dequant(q, absmax, codebook, o, m, k)` (extension.cpp:40-49); o fp16 [m,k]."""
    dev = q.device if isinstance(q, torch.Tensor) else None
    _expect(q, "q", torch.uint8, m * k // 2)
    _expect(absmax, "absmax", torch.float32, m, dev)
    _expect(codebook, "codebook", torch.float32, 16, dev)
    _expect(o, "o", torch.float16, m * k, dev)
    with torch.cuda.device(dev):
        check(_lib.load().tuna_dequant(q.data_ptr(), absmax.data_ptr(), codebook.data_ptr(), o.data_ptr(),
                                       m, k, _stream_ptr(dev)))


def quantize(w, codebook=None):
    """Row-wise absmax quantizer + packer on the device: the reference's
    `quantize_blockwise_dynamic_4bit(w, block_size=k, preprocess=True)` (test.py:7-68) with the
    same return structure `(q, (absmax, code))`: `q` uint8 `[m/8, k/8, 32]`, `absmax` fp32 `[m]`,
    `code` fp32 `[16]` (NF4 unless `codebook` is given)."""
    from .codebooks import nf4_tensor

    if not isinstance(w, torch.Tensor) or not w.is_cuda:
        raise ValueError("w must be a CUDA tensor (there is no CPU path)")
    if w.dtype != torch.float16 or w.dim() != 2 or not w.is_contiguous():
        raise ValueError("w must be a contiguous fp16 [m, k] tensor")
    m, k = w.shape
    code = nf4_tensor(w.device) if codebook is None else codebook
    _expect(code, "codebook", torch.float32, 16, w.device)
    q = torch.empty((m // 8, k // 8, 32), dtype=torch.uint8, device=w.device)
    absmax = torch.empty((m,), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        check(_lib.load().tuna_quantize(w.data_ptr(), code.data_ptr(), q.data_ptr(), absmax.data_ptr(), m, k,
                                        _stream_ptr(w.device)))
    return q, (absmax, code)


class HostPipeline:
    """`matmul` for callers whose activations and outputs live in (pinned) HOST memory, with the
    copies overlapped with the GEMMs of neighbouring calls.

    Each call copies `x_host` to a device staging slot on a copy-in stream, runs the GEMM on
    the caller's current stream, and copies the result to `o_host` on a copy-out stream; events
    order the three and guard the reuse of the `depth` staging slots.  Calls return at once;
    `join()` makes the current stream wait for every outstanding copy-out (call it before
    reading `o_host` buffers, followed by a stream or event synchronisation).  Weights, scales
    and codebook are parameters and stay on the device, as in the reference.

    A sequence `begin(); matmul(...); ...; join()` can be captured into a CUDA graph (the host
    buffers are then fixed addresses read and written at every replay): `begin()` forks the two
    copy streams off the capturing stream and forgets slot history from before the capture.
    """

    def __init__(self, device, max_x_elems: int, max_o_elems: int, depth: int = 4):
        self.device = torch.device(device)
        self.depth = int(depth)
        self.copy_in = torch.cuda.Stream(device=self.device)
        self.copy_out = torch.cuda.Stream(device=self.device)
        self._slots = []
        for _ in range(self.depth):
            self._slots.append({
                "x": torch.empty(max_x_elems, dtype=torch.float16, device=self.device),
                "o": torch.empty(max_o_elems, dtype=torch.float16, device=self.device),
                "in": torch.cuda.Event(), "gemm": torch.cuda.Event(), "out": torch.cuda.Event(), "used": False,
            })
        self._next = 0
        self._fork = torch.cuda.Event()
        # the staging memory was allocated on the current stream
        self.copy_in.wait_stream(torch.cuda.current_stream(self.device))
        self.copy_out.wait_stream(torch.cuda.current_stream(self.device))

    def matmul(self, x_host, q, s, c, o_host, m: int, n: int, k: int, *, workspace=None, after_gemm=None) -> None:
        """One GEMM with host activations and output.  `after_gemm(o_dev)` (optional) runs on the
        compute stream between the GEMM and the copy-out (e.g. an all-reduce of a K-split layer)."""
        if n * k > self._slots[0]["x"].numel() or n * m > self._slots[0]["o"].numel():
            raise ValueError("HostPipeline staging slots are smaller than this GEMM's activations or output")
        if not (x_host.is_pinned() and o_host.is_pinned()):
            raise ValueError("HostPipeline needs pinned host tensors (pageable copies would serialise)")
        slot = self._slots[self._next % self.depth]
        self._next += 1
        compute = torch.cuda.current_stream(self.device)
        xd = slot["x"][: n * k].view(n, k)
        od = slot["o"][: n * m].view(n, m)
        if slot["used"]:
            self.copy_in.wait_event(slot["gemm"])  # the slot's previous GEMM has read its activations
        with torch.cuda.stream(self.copy_in):
            xd.copy_(x_host, non_blocking=True)
            slot["in"].record(self.copy_in)
        compute.wait_event(slot["in"])
        if slot["used"]:
            compute.wait_event(slot["out"])        # the slot's previous result has left the device
        matmul(xd, q, s, c, od, m, n, k, workspace=workspace)
        if after_gemm is not None:
            after_gemm(od)
        slot["gemm"].record(compute)
        self.copy_out.wait_event(slot["gemm"])
        with torch.cuda.stream(self.copy_out):
            o_host.copy_(od, non_blocking=True)
            slot["out"].record(self.copy_out)
        slot["used"] = True

    def begin(self) -> None:
        """Start of a sequence: both copy streams wait for the current stream's work so far, and
        the staging slots are treated as free (their earlier uses are ordered before that point)."""
        compute = torch.cuda.current_stream(self.device)
        self.join()
        self._fork.record(compute)
        self.copy_in.wait_event(self._fork)
        self.copy_out.wait_event(self._fork)
        for slot in self._slots:
            slot["used"] = False
        self._next = 0

    def reset(self) -> None:
        """Forget every earlier use of the staging slots.  Only when the device is idle (after a
        synchronisation), e.g. right before capturing a sequence into a CUDA graph."""
        for slot in self._slots:
            slot["used"] = False
        self._next = 0

    def join(self) -> None:
        """The current stream waits for every copy-out issued so far."""
        compute = torch.cuda.current_stream(self.device)
        for slot in self._slots:
            if slot["used"]:
                compute.wait_event(slot["out"])
