"""Gradient exchange on the copy engines: an average over the ranks of one node built from peer-to-peer copies and a
few element-wise kernels, for trainers whose backward pass is made of persistent kernels.  A collective that runs on
SMs (NCCL) holds its CTAs' SMs for as long as it lasts, and a GEMM CTA with over 200 KB of shared memory cannot share an
SM with them; copies issued with ``cudaMemcpyAsync`` between peer-mapped buffers run on the DMA engines and leave every
SM to the backward pass.

Every rank exports the buffers that take part (``Tensor.untyped_storage()._share_cuda_()``, a CUDA IPC handle), opens
its peers' (``sp24_ipc_open``) and then, per exchanged range, (1) waits until all ranks have their values ready,
(2) pulls its own shard of the range from every peer and sums, (3) waits until all ranks have summed, (4) pulls the
other shards, already averaged, from their owners.  The waits are one-element NCCL all-reduces on the exchange stream:
when one completes on a rank, every rank's exchange stream has reached it.  Nothing here waits in a kernel of its own.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _ext


class _DevicePointer:
    """A raw device address as something ``torch.as_tensor`` accepts (bytes; view it in the wanted dtype)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerBuffers:
    """``tensor`` (contiguous, CUDA) of every rank of the process group, as tensors on this rank's device: entry
    ``[rank]`` is the local tensor, the others alias the peers' memory.  All ranks must call this together."""

    def __init__(self, tensor: torch.Tensor, group=None):
        _ext.require_cuda(tensor)
        if not tensor.is_contiguous():
            raise RuntimeError("PeerBuffers: contiguous tensors only")
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.local = tensor
        storage = tensor.untyped_storage()
        shared = storage._share_cuda_()
        handle, offset = bytes(shared[1]), int(shared[3])
        # The framework counts references of a shared block on behalf of consumers that rebuild it through its own
        # machinery; the peers here map the block themselves and are held off by close() + a barrier instead, so the
        # count taken by the call above is handed straight back (otherwise the block would stay parked until exit).
        try:
            type(storage)._release_ipc_counter(shared[4], shared[5], device=shared[0])
        except Exception:    # a torch without this hook: the block is released at process exit
            pass
        # newer torch puts a version byte and a type byte ('c': plain cudaMalloc block, 'e': expandable segment) in
        # front of the 64 bytes of the cudaIpcMemHandle_t
        if len(handle) == 66 and handle[1:2] == b"c":
            handle = handle[2:]
        if len(handle) != 64:
            raise RuntimeError(f"PeerBuffers: unsupported storage handle ({len(handle)} bytes, prefix {handle[:2]!r}); "
                               "allocate the buffer without expandable segments")
        offset += tensor.storage_offset() * tensor.element_size()
        infos = [None] * self.world
        dist.all_gather_object(infos, (handle, offset, tensor.numel(), str(tensor.dtype)), group=group)
        self._opened = []
        self.views = []
        for p, (h, off, numel, dtype) in enumerate(infos):
            if numel != tensor.numel() or dtype != str(tensor.dtype):
                raise RuntimeError("PeerBuffers: the ranks' tensors differ in size or dtype")
            if p == self.rank:
                self.views.append(tensor.view(-1))
                continue
            base = ctypes.c_void_p()
            _ext.check(_ext.lib().sp24_ipc_open(h, len(h), ctypes.byref(base)), "sp24_ipc_open")
            self._opened.append(base.value)
            raw = torch.as_tensor(_DevicePointer(base.value + off, numel * tensor.element_size()), device=tensor.device)
            self.views.append(raw.view(tensor.dtype))

    def close(self):
        self.views = []
        for ptr in self._opened:
            _ext.lib().sp24_ipc_close(ptr)
        self._opened = []


class CopyEngineAverage:
    """Averages ranges of registered buffers over the ranks.  ``add_buffer(name, tensor)`` on every rank (same order),
    then ``average(name, a, b)`` for element ranges [a, b), all ranks in the same order, on the stream the caller has
    made current; ``finish()`` once after the last range of a step, before any rank overwrites a registered buffer."""

    def __init__(self, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.buffers = {}
        self._flag = None
        self._stage = {}
        # one side stream per peer: the copies of a phase come from different peers over different links and run on
        # different copy engines side by side; issued on one stream they would queue behind one another
        self._side = None
        self._fork = None
        self._join = None

    def add_buffer(self, name, tensor: torch.Tensor):
        self.buffers[name] = PeerBuffers(tensor, self.group)
        if self._flag is None:
            self._flag = torch.zeros(1, dtype=torch.float32, device=tensor.device)

    def _barrier(self):
        dist.all_reduce(self._flag, group=self.group)

    def _parallel_copies(self, pairs):
        """dst.copy_(src) for every (dst, src) of ``pairs``, each on its own side stream, forked from and joined to the
        current stream."""
        pairs = [pr for pr in pairs if pr[0].numel() > 0]
        if not pairs:
            return
        cur = torch.cuda.current_stream()
        if len(pairs) == 1:
            pairs[0][0].copy_(pairs[0][1])
            return
        if self._side is None:
            self._side = [torch.cuda.Stream() for _ in range(self.world - 1)]
            self._fork = torch.cuda.Event()
            self._join = [torch.cuda.Event() for _ in range(self.world - 1)]
        self._fork.record(cur)
        for i, (dst, src) in enumerate(pairs):
            st = self._side[i % len(self._side)]
            st.wait_event(self._fork)
            with torch.cuda.stream(st):
                dst.copy_(src)
                self._join[i % len(self._side)].record(st)
        for i in range(min(len(pairs), len(self._side))):
            cur.wait_event(self._join[i])

    def _shard(self, a, b, p):
        per = -(-(b - a) // self.world)
        per = (per + 7) // 8 * 8                       # 16-byte pieces for 16-bit types, 32-byte ones for float32
        lo = min(b, a + p * per)
        return lo, min(b, lo + per)

    def average(self, name, a, b):
        pb = self.buffers[name]
        mine = pb.views[self.rank]
        lo, hi = self._shard(a, b, self.rank)
        n = hi - lo
        key = (name, mine.dtype)
        need = max(self._shard(a, b, 0)[1] - a, 1)
        st = self._stage.get(key)
        if st is None or st.shape[1] < need:
            st = torch.empty((self.world - 1, need), dtype=mine.dtype, device=mine.device)
            self._stage[key] = st
        self._barrier()                                  # every rank's values of [a, b) are complete
        if n > 0:
            others = [p for p in range(self.world) if p != self.rank]
            self._parallel_copies([(st[i, :n], pb.views[p][lo:hi]) for i, p in enumerate(others)])   # DMA, no SM
            if mine.dtype == torch.float32:
                acc = mine[lo:hi]
                for i in range(len(others)):
                    acc.add_(st[i, :n])
                acc.mul_(1.0 / self.world)
            else:                                        # 16-bit values are summed in float32
                acc = mine[lo:hi].float()
                for i in range(len(others)):
                    acc.add_(st[i, :n])
                mine[lo:hi].copy_(acc.mul_(1.0 / self.world))
        self._barrier()                                  # every rank's shard is averaged
        pulls = []
        for p in range(self.world):
            if p != self.rank:
                plo, phi = self._shard(a, b, p)
                pulls.append((mine[plo:phi], pb.views[p][plo:phi]))
        self._parallel_copies(pulls)

    def finish(self):
        self._barrier()                                  # every rank has pulled what it needs from the others

    def close(self):
        for pb in self.buffers.values():
            pb.close()
        self.buffers = {}
