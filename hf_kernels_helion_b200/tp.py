"""Column-parallel (N-sharded) block-FP8 linear over the GPUs of one node.

The reference has no multi-GPU code; this layer follows directly from its kernel's
data dependence (torch-ext/finegrained_fp8_helion/fp8.py:30-36): an output column
block ``C[:, n0:n1]`` reads only rows ``n0:n1`` of ``B`` and rows ``n0/128:n1/128`` of
``Bs``, while ``A`` / ``As`` are used whole.  So rank r keeps the r-th slice of the
weight's N rows, every rank computes its column slice of C with the single-GPU
kernel, and ONE all-gather of the bf16 slices over NCCL / NVLink assembles [M, N].

One process per GPU (torchrun); ``torch.distributed`` must be initialised.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_bounds(N: int, world: int, rank: int, block_n: int = 128):
    """Rows [n0, n1) of the weight that `rank` owns.  N must split into `world` equal
    slices that are whole 128-row scale blocks."""
    if N % (world * block_n) != 0:
        raise ValueError(f"N = {N} must be a multiple of world_size * {block_n} = {world * block_n}")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_weight(B: torch.Tensor, Bs: torch.Tensor, world: int, rank: int, block_n: int = 128):
    """Slice a full block-FP8 weight ``B [N, K]`` / ``Bs [N/128, K/128]`` for `rank`."""
    n0, n1 = shard_bounds(B.shape[0], world, rank, block_n)
    return B[n0:n1], Bs[n0 // block_n:n1 // block_n]


# A CUDA IPC handle names a whole allocation and may be opened only once per process: buffers
# that the caching allocator carved out of one segment share a handle, so mappings are kept
# here by handle bytes with a use count.
_ipc_mappings: dict = {}


def _ipc_open_shared(lib, handle: bytes) -> int:
    import ctypes

    from . import _lib

    entry = _ipc_mappings.get(handle)
    if entry is None:
        base = ctypes.c_void_p(0)
        _lib.check(lib.b200fp8_ipc_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(base)), "b200fp8_ipc_open")
        entry = [int(base.value), 0]
        _ipc_mappings[handle] = entry
    entry[1] += 1
    return entry[0]


def _ipc_close_shared(lib, handle: bytes) -> None:
    import ctypes

    entry = _ipc_mappings.get(handle)
    if entry is None:
        return
    entry[1] -= 1
    if entry[1] <= 0:
        lib.b200fp8_ipc_close(ctypes.c_void_p(entry[0]))
        del _ipc_mappings[handle]


class PeerBuffers:
    """One [M, N] output buffer per rank, each mapped into every process of the group
    (CUDA IPC), so that a kernel on any GPU can store into all of them over NVLink.
    ptr(r) is the device address, valid in THIS process, of rank r's buffer."""

    def __init__(self, M: int, N: int, dtype: torch.dtype, device: torch.device, group=None):
        import ctypes

        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        # one allocation: the [M, N] buffer followed by a 256-byte tail that holds this rank's eight
        # barrier flags (zero at start), so that one IPC mapping gives the peers both
        esize = torch.empty((), dtype=dtype).element_size()
        self._body = -(-(M * N * esize) // 256) * 256
        raw = torch.empty(self._body + 256, dtype=torch.uint8, device=device)
        raw[self._body:].zero_()
        self.local = raw[:M * N * esize].view(dtype).view(M, N)
        self.flags = raw[self._body:self._body + 32].view(torch.int32)
        self._raw = raw
        lib = _lib.load()
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_int64(0)
        with torch.cuda.device(device):
            _lib.check(lib.b200fp8_ipc_export(self.local.data_ptr(), handle, ctypes.byref(offset)), "b200fp8_ipc_export")
            metas = [None] * self.world
            dist.all_gather_object(metas, (bytes(handle.raw), int(offset.value)), group=group)
            self._bases = {}
            self._ptrs = [0] * self.world
            for r, (h, off) in enumerate(metas):
                if r == self.rank:
                    self._ptrs[r] = self.local.data_ptr()
                    continue
                self._bases[r] = h
                self._ptrs[r] = _ipc_open_shared(lib, h) + off
        dist.barrier(group)

    def ptr(self, r: int) -> int:
        return self._ptrs[r]

    def flag_ptr(self, r: int) -> int:
        """Device address, valid in this process, of rank r's barrier flag array."""
        return self._ptrs[r] + self._body

    def barrier(self, epoch: int) -> None:
        """Enqueue the device-side barrier (b200fp8_peer_barrier) on the current stream: work queued
        behind it sees what every rank's kernels queued before their barrier of the same epoch wrote."""
        import ctypes

        from . import _lib, runtime

        dev = self.local.device
        arr = (ctypes.c_void_p * self.world)(*[self.flag_ptr(r) for r in range(self.world)])
        with torch.cuda.device(dev):
            st = _lib.load().b200fp8_peer_barrier(arr, self.world, self.rank, epoch & 0xFFFFFFFF,
                                                  runtime.status_word(dev).data_ptr(),
                                                  torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(st, "b200fp8_peer_barrier")

    def close(self) -> None:
        from . import _lib

        torch.cuda.synchronize()
        dist.barrier(self.group)          # nobody may still be storing into a buffer that is about to be unmapped
        lib = _lib.load()
        for h in self._bases.values():
            _ipc_close_shared(lib, h)
        self._bases = {}


def multicast_supported(device: torch.device) -> bool:
    """True when the CUDA driver reports NVLink multicast support for this device (what torch's
    symmetric memory needs to hand out a multicast address)."""
    try:
        from torch._C._autograd import DeviceType
        from torch._C._distributed_c10d import _SymmetricMemory
        return bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, device.index or 0))
    except Exception:  # noqa: BLE001 - any failure of the probe means "do not use it"
        return False


class MulticastBuffers:
    """One [M, N] output buffer per rank in torch symmetric memory, bound to an NVLink multicast
    object: a store to `mc_ptr + offset` (multimem.st) lands at `offset` in EVERY rank's buffer,
    replicated by the NVSwitch. `local` is this rank's copy as a tensor. Raises RuntimeError
    where the group has no multicast support (mc_ptr would be 0)."""

    def __init__(self, M: int, N: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.local = symm_mem.empty((M, N), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.local, group=self.group)
        mc_base = int(self.handle.multicast_ptr)
        if mc_base == 0:
            raise RuntimeError("symmetric memory rendezvous gave no multicast address (NVLink multicast unsupported here)")
        # the handle describes the allocation the tensor lives in: carry the tensor's offset over
        rank = dist.get_rank(self.group)
        offset = self.local.data_ptr() - int(self.handle.buffer_ptrs[rank])
        nbytes = M * N * self.local.element_size()
        if offset < 0 or offset + nbytes > int(self.handle.buffer_size):
            raise RuntimeError("symmetric memory handle does not cover the tensor it was made for")
        self.mc_ptr = mc_base + offset
        dist.barrier(self.group)


class ShardedFp8Linear:
    """Holds this rank's weight slice and runs  C = A . B^T  tensor-parallel.

    matmul: callable ``(A, B, As, Bs, block_size, output_dtype) -> [M, N_local]``;
    defaults to the package's CUDA op.  (The CPU tests inject a checker here to
    exercise the sharding and gather logic under gloo without a GPU.)
    """

    def __init__(self, B_local: torch.Tensor, Bs_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 matmul: Optional[Callable] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.B, self.Bs = B_local, Bs_local
        self.n_local = B_local.shape[0]
        if self.n_local % 128 != 0:
            raise ValueError("the local weight slice must be a whole number of 128-row blocks")
        self._injected = matmul is not None
        self.matmul = matmul
        # forward_fused: True = the ranks meet in a one-warp kernel that exchanges flags over NVLink
        # (b200fp8_peer_barrier); False = a one-element NCCL all-reduce plays the barrier
        self.device_barrier = True
        self._gather_buf = None

    @classmethod
    def from_full(cls, B: torch.Tensor, Bs: torch.Tensor, group=None, matmul=None) -> "ShardedFp8Linear":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        b, bs = shard_weight(B, Bs, world, rank)
        return cls(b.contiguous(), bs.contiguous(), group, matmul)

    @property
    def N(self) -> int:
        return self.n_local * self.world

    def _buffer(self, M: int, dtype, device) -> torch.Tensor:
        b = self._gather_buf
        if b is None or b.shape[1] != M or b.dtype != dtype or b.device != device:
            b = torch.empty((self.world, M, self.n_local), dtype=dtype, device=device)
            self._gather_buf = b
        return b

    def local(self, A: torch.Tensor, As: torch.Tensor, output_dtype=torch.bfloat16, out=None) -> torch.Tensor:
        """This rank's column slice C[:, n0:n1] (no communication), written into `out` if given."""
        if self._injected:
            res = self.matmul(A, self.B, As, self.Bs, [128, 128], output_dtype)
            if out is None:
                return res
            out.copy_(res)
            return out
        from . import runtime  # noqa: PLC0415
        return runtime.gemm(A, self.B, As, self.Bs, 128, 128, output_dtype, out=out)

    def forward_slots(self, A: torch.Tensor, As: torch.Tensor, output_dtype=torch.bfloat16) -> torch.Tensor:
        """Compute and all-gather; returns the gather buffer [world, M, N/world] whose slot r
        is rank r's column slice.  ``slots.permute(1, 0, 2)`` is a zero-copy [M, world, N/world]
        view holding the same values as C[M, N].  The GEMM writes straight into this rank's
        slot and the all-gather runs in place, so the only extra traffic is the gather itself."""
        buf = self._buffer(A.shape[0], output_dtype, A.device)
        mine = buf[self.rank]
        self.local(A, As, output_dtype, out=mine)
        if self.world > 1:
            dist.all_gather_into_tensor(buf.view(-1), mine.reshape(-1), group=self.group)
        return buf

    def forward_fused(self, A: torch.Tensor, As: torch.Tensor, output_dtype=torch.bfloat16,
                      reader_done: Optional[torch.cuda.Event] = None) -> torch.Tensor:
        """Contiguous C [M, N] on every rank with the exchange fused into the GEMM: the kernel's
        epilogue stores this rank's column slice into the [M, N] buffer of EVERY rank (peer
        stores over NVLink), and a one-warp flag-exchange kernel afterwards (or, with
        device_barrier = False, one tiny all-reduce) is the barrier that tells each rank that all
        slices have arrived.  No all-gather, no transpose copy, no NCCL call on the data path.

        Two buffer sets alternate between calls: the result returned by call i stays valid until
        call i + 2 is issued.  Peers start overwriting that buffer once THIS rank has passed the
        barrier of call i + 1, so every reader of call i's result must be ordered before that
        barrier: work enqueued on the current stream before call i + 1 is; a reader on ANOTHER
        stream (a read-back on a copy stream, say) must record an event when it is done and pass
        it as `reader_done` to call i + 1, which makes the current stream wait for it before the
        barrier is enqueued."""
        from . import runtime  # noqa: PLC0415

        M = A.shape[0]
        key = (M, output_dtype, A.device)
        if getattr(self, "_peer_key", None) != key:
            for pb in getattr(self, "_peer", []):
                pb.close()
            self._peer = [PeerBuffers(M, self.N, output_dtype, A.device, self.group) for _ in range(2)]
            self._peer_key = key
            self._peer_turn = 0
            self._epoch = 0
            self._flag = torch.zeros(1, dtype=torch.float32, device=A.device)
        pb = self._peer[self._peer_turn]
        self._peer_turn ^= 1
        esize = pb.local.element_size()
        col_bytes = self.rank * self.n_local * esize
        # start the remote stores at different peers on different ranks
        order = [self.rank] + [(self.rank + i) % self.world for i in range(1, self.world)]
        ptrs = [pb.ptr(r) + col_bytes for r in order]
        runtime.gemm_scatter(A, self.B, As, self.Bs, ptrs, [self.N] * self.world, output_dtype)
        if reader_done is not None:
            torch.cuda.current_stream(A.device).wait_event(reader_done)
        if self.world > 1:
            if self.device_barrier:
                self._epoch += 1
                self._peer[0].barrier(self._epoch)      # one flag set serves both buffer sets
            else:
                dist.all_reduce(self._flag, group=self.group)
        return pb.local

    def forward_multimem(self, A: torch.Tensor, As: torch.Tensor, output_dtype=torch.bfloat16) -> torch.Tensor:
        """Contiguous C [M, N] on every rank, exchange fused into the GEMM through NVLink multicast:
        the epilogue writes this rank's column slice ONCE to the multicast view of the [M, N]
        buffers and the NVSwitch replicates it into every rank's copy, so a GPU sends N/world
        columns instead of (world - 1) x that. One tiny all-reduce afterwards is the barrier.
        Buffer alternation and lifetime of the returned tensor as for forward_fused."""
        from . import runtime  # noqa: PLC0415

        M = A.shape[0]
        key = (M, output_dtype, A.device)
        if getattr(self, "_mc_key", None) != key:
            self._mc = [MulticastBuffers(M, self.N, output_dtype, A.device, self.group) for _ in range(2)]
            self._mc_key = key
            self._mc_turn = 0
            self._mc_flag = torch.zeros(1, dtype=torch.float32, device=A.device)
        mb = self._mc[self._mc_turn]
        self._mc_turn ^= 1
        col_bytes = self.rank * self.n_local * mb.local.element_size()
        runtime.gemm_multicast(A, self.B, As, self.Bs, mb.mc_ptr + col_bytes, self.N, output_dtype)
        if self.world > 1:
            dist.all_reduce(self._mc_flag, group=self.group)
        return mb.local

    def forward(self, A: torch.Tensor, As: torch.Tensor, output_dtype=torch.bfloat16) -> torch.Tensor:
        """Contiguous C [M, N] on every rank (all-gather, then one transpose copy of the slots)."""
        slots = self.forward_slots(A, As, output_dtype)
        M = A.shape[0]
        return slots.permute(1, 0, 2).reshape(M, self.N)

    __call__ = forward
