"""Peer-memory communicator of the tensor-parallel decoder: one symmetric buffer per rank, mapped
into every peer (two data slots with one receive region per source rank), and the fused
`all-reduce + residual add + RMS norm` kernel that runs on it: every rank stores its partial, the
call's epoch attached to every 4 bytes, into its region of every peer's buffer, polls its own
regions until the epochs are in place, and reduces from local memory
(C ABI: the qfb_comm_* entry points of include/qfactory_b200.h).

It takes the place of the collective call after a row-parallel linear in the reference's serving
stack (reference: third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:1100-1124) for the
small messages of a decode step, as that stack's own one-shot kernel does (reference:
third_party/vllm-bitblas/vllm/distributed/device_communicators/custom_all_reduce.py:242-255).
Larger messages (a prefill) stay on the process group's all-reduce.

The buffers are exchanged as CUDA IPC handles over the process group at construction; after that
no host communication is involved and the kernels are CUDA-graph safe.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _native


class _DevView:
    """A device address exposed through the CUDA array interface, so that torch can alias it."""

    def __init__(self, ptr, shape, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f2", "data": (int(ptr), False), "version": 3,
                                         "strides": None}
        self._owner = owner


class PeerComm:
    """`world` symmetric buffers with two data slots of `slot_rows x d` fp16 each.

    `PeerComm.from_process_group(d, slot_rows, group)` builds one over the ranks of a process group
    (one process per GPU of one node).  `PeerComm.local_emulation(...)` builds the `world` buffers
    of all ranks inside ONE process on one GPU, for tests that play a peer's part by hand
    (`write_peer_partial`).
    """

    def __init__(self, rank, world, bases, d, slot_rows, device, owned=None, opened=()):
        L = _native.lib()
        self._lib, self.rank, self.world, self.d, self.device = L, rank, world, d, device
        self.slot_rows = min(slot_rows, L.qfb_comm_max_rows())
        self.slot_bytes = self.slot_rows * d * 2
        self.bases = list(bases)
        self._owned, self._opened = owned, list(opened)
        arr = (ctypes.c_void_p * world)(*self.bases)
        h = ctypes.c_void_p()
        with torch.cuda.device(device):
            _native.check(L.qfb_comm_create(rank, world, arr, self.slot_bytes, ctypes.byref(h)), "qfb_comm_create")
        self._h = h
        self._slots = [torch.as_tensor(_DevView(L.qfb_comm_slot(h, s), (self.slot_rows, d), self), device=device)
                       for s in (0, 1)]
        self._next = 0

    # -- construction -----------------------------------------------------------
    @staticmethod
    def _alloc(slot_bytes, device):
        L = _native.lib()
        base, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            _native.check(L.qfb_comm_alloc(slot_bytes, ctypes.byref(base), handle), "qfb_comm_alloc")
        return base.value, handle.raw

    @classmethod
    def from_process_group(cls, d, slot_rows, device, group=None):
        L = _native.lib()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        slot_rows = min(slot_rows, L.qfb_comm_max_rows())
        base, handle = cls._alloc(slot_rows * d * 2, device)
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        bases, opened = [], []
        with torch.cuda.device(device):
            for r in range(world):
                if r == rank:
                    bases.append(base)
                    continue
                p = ctypes.c_void_p()
                _native.check(L.qfb_comm_open(handles[r], ctypes.byref(p)), f"qfb_comm_open(rank {r})")
                bases.append(p.value)
                opened.append(p.value)
        comm = cls(rank, world, bases, d, slot_rows, device, owned=base, opened=opened)
        dist.barrier(group)   # every rank has mapped every buffer before anyone raises a flag
        try:
            comm.self_check(group)
        except Exception:
            comm.close()
            raise
        return comm

    def self_check(self, group=None) -> None:
        """One reduction per slot on a known pattern with a short wait limit, compared with the sum
        it must give; every rank raises if any rank saw a wrong sum or a wait that ran out, so that
        a node whose peer mappings do not carry stores is found at construction, not in the middle
        of a decode step."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group)                      # all ranks enter together: the short limit below is safe
        rows = min(2, self.slot_rows)
        self.set_timeout_us(500_000)
        good = True
        try:
            for which in (0, 1):
                col = torch.arange(self.d, device=self.device, dtype=torch.float32) % 7
                self.slot(which, rows).copy_(((self.rank + 1) * (col + 1) / 8).half().expand(rows, self.d))
                got = self.allreduce_add_rmsnorm(which, None, None, rows)
                want = (self.world * (self.world + 1) / 2 * (col + 1) / 8).half().expand(rows, self.d)
                torch.cuda.synchronize(self.device)
                good = good and bool(torch.equal(got, want))
            good = good and self.read_status() == 0
        finally:
            self.set_timeout_us(2_000_000)
        ok = torch.tensor([1 if good else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok[0]) == 0:
            raise RuntimeError("peer-memory reduction self-check failed" + ("" if good else " on this rank"))

    @classmethod
    def local_emulation(cls, rank, world, d, slot_rows, device="cuda"):
        """All `world` buffers allocated by this process on one GPU; returns the communicator of
        `rank`.  `write_peer_partial(r, slot, t)` lets a test put a peer's partial in place before
        the kernel is launched (the kernel of a second rank is never run beside this one on the same
        GPU: kernels that wait on one another must not share a GPU)."""
        L = _native.lib()
        device = torch.device(device)
        slot_rows = min(slot_rows, L.qfb_comm_max_rows())
        bases = [cls._alloc(slot_rows * d * 2, device)[0] for _ in range(world)]
        comm = cls(rank, world, bases, d, slot_rows, device, owned=None, opened=())
        comm._emulated = bases
        return comm

    # -- use ----------------------------------------------------------------------
    def slot(self, which: int, rows: int) -> torch.Tensor:
        """fp16 [rows, d] view of the local data slot `which` (the row-parallel linear's `out=`)."""
        return self._slots[which][:rows]

    def next_slot(self) -> int:
        """Slots must alternate between consecutive reductions; this hands out 0, 1, 0, ..."""
        s = self._next
        self._next ^= 1
        return s

    def fits(self, rows: int, d: int) -> bool:
        return d == self.d and 0 < rows <= self.slot_rows

    # -- step numbering: the exchange whose receiving side may be the GEMV that consumes the sum -------------
    def step_begin(self) -> None:
        """Advance the step counter (one tiny launch; every rank, once per decode step, before its first
        reduction).  Reduction `idx` of the step then carries the epoch 2^31 | step << 8 | idx."""
        _native.check(self._lib.qfb_comm_step_begin(self._h, torch.cuda.current_stream(self.device).cuda_stream),
                      "qfb_comm_step_begin")

    def step_epoch(self, idx: int) -> int:
        """The epoch reduction `idx` of the current step uses (synchronises; tests)."""
        torch.cuda.synchronize(self.device)
        words = torch.as_tensor(_DevView(self.bases[self.rank], (1, 512), self), device=self.device).view(torch.int32)
        return (0x80000000 | ((int(words[0, 65]) & 0x7FFFFF) << 8) | idx) & 0xFFFFFFFF

    def collect_norm_linear(self, layer, which, idx, x, x_out, norm_weight, rows, eps=1e-5, out=None):
        """y = (rmsnorm(x + sum over the ranks of slot `which`) * norm_weight) @ dequant(W)^T in ONE kernel: the
        GEMV collects the partials (its own from the slot, the peers' from what they sent for reduction `idx`
        of this step) while it stages its activations; x + sum goes to `x_out` (another buffer than `x`)."""
        if out is None:
            out = torch.empty(rows, layer.out_features, dtype=torch.float16, device=self.device)
        if layer._desc is None:
            layer._prepare()
        st = self._lib.qfb_linear_collect_addnorm_forward(
            layer._desc_ref, self._h, which, idx, x.data_ptr(), None if x_out is None else x_out.data_ptr(),
            norm_weight.data_ptr(), float(eps), rows, out.data_ptr(), layer._ws_ptr, layer._ws_bytes, layer.flags,
            torch.cuda.current_stream(self.device).cuda_stream)
        _native.check(st, "qfb_linear_collect_addnorm_forward")
        return out

    def collect_supported(self, sender, receiver, rows: int) -> bool:
        """True when `sender` (a row-parallel layer) can send its partial itself and `receiver` (the layer that
        consumes the normed sum; None: the reduction kernel) can collect it, for `rows` batch rows."""
        from . import layout as _layout

        def ok4(l):
            return l.packed_layout == _layout.LAYOUT_FRAGMENT and l.n_bits == 4 and l.group_size != 64
        if not (0 < rows <= 16 and ok4(sender) and sender.out_features == self.d and self.d % 128 == 0):
            return False
        if receiver is None:
            return True
        if not (ok4(receiver) and receiver.in_features == self.d):
            return False
        if receiver._desc is None:
            receiver._prepare()
        return bool(self._lib.qfb_linear_addnorm_supported(receiver._desc_ref, rows))

    def linear_into_slot(self, layer, x, which, rows, silu_mul=False, push=True, idx=None) -> bool:
        """Run the row-parallel `layer` on `x` ([rows, k], or the fused gate/up tensor [rows, 2k] with
        `silu_mul`) with data slot `which` as its output.  Returns True when the kernel also sent the
        partial to the peers while storing it (one launch for the linear and the first half of the
        reduction; reference: matmul, then a collective call,
        third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:1100-1124): the reduction must
        then be called with `pushed=True`.  Where that kernel does not serve the layer or the batch,
        the plain forward runs with the slot as `out=` and False is returned."""
        if push and layer.out_features == self.d and 0 < rows <= 16:
            if layer._desc is None:
                layer._prepare()
            x2 = x.reshape(rows, -1)
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            if (not silu_mul) or layer.silu_mul_supported(rows):
                stream = torch.cuda.current_stream(self.device).cuda_stream
                if idx is None:
                    fn = self._lib.qfb_linear_silu_mul_forward_reduce if silu_mul else self._lib.qfb_linear_forward_reduce
                    st = fn(layer._desc_ref, x2.data_ptr(), rows, self._h, which, layer._ws_ptr, layer._ws_bytes, layer.flags, stream)
                else:   # step numbering: the receiver waits for exactly this epoch, so there is no fallback
                    fn = (self._lib.qfb_linear_silu_mul_forward_reduce_step if silu_mul
                          else self._lib.qfb_linear_forward_reduce_step)
                    st = fn(layer._desc_ref, x2.data_ptr(), rows, self._h, which, idx, layer._ws_ptr, layer._ws_bytes,
                            layer.flags, stream)
                    _native.check(st, "qfb_linear_forward_reduce_step")
                if st == 0:
                    return True
                if st != 3:   # QFB_ERR_UNSUPPORTED: fall through to the two-step form
                    _native.check(st, "qfb_linear_forward_reduce")
        assert idx is None, "a step-numbered reduction needs the sending GEMV (collect_supported says when it serves)"
        if silu_mul:
            layer.forward_silu_mul(x, out=self.slot(which, rows))
        else:
            layer(x, out=self.slot(which, rows))
        return False

    def allreduce_add_rmsnorm(self, which, x, weight, rows, eps=1e-5, out=None, pushed=False, idx=None):
        """Sum slot `which` over the ranks; `x` (fp16 [rows, d], may be None) += the sum in place;
        returns the RMS norm of the row with `weight` (or the row itself when `weight` is None).
        `pushed`: the partial was already sent to the peers (`linear_into_slot` returned True)."""
        if out is None:
            out = torch.empty(rows, self.d, dtype=torch.float16, device=self.device)
        if idx is not None:   # step numbering: collects what the sending GEMVs stamped with reduction `idx` of this step
            st = self._lib.qfb_allreduce_add_rmsnorm_step(
                self._h, which, idx, None if x is None else x.data_ptr(), None if weight is None else weight.data_ptr(),
                out.data_ptr(), rows, self.d, eps, torch.cuda.current_stream(self.device).cuda_stream)
            if st != 0:
                _native.check(st, "qfb_allreduce_add_rmsnorm_step")
            return out
        fn = self._lib.qfb_allreduce_add_rmsnorm_pushed if pushed else self._lib.qfb_allreduce_add_rmsnorm
        st = fn(
            self._h, which, None if x is None else x.data_ptr(), None if weight is None else weight.data_ptr(),
            out.data_ptr(), rows, self.d, eps, torch.cuda.current_stream(self.device).cuda_stream)
        if st != 0:
            _native.check(st, "qfb_allreduce_add_rmsnorm")
        return out

    def set_timeout_us(self, us: int) -> None:
        self._lib.qfb_comm_set_timeout_us(self._h, us)

    def read_status(self) -> int:
        """0, or 8 (QFB_ERR_DEVICE_FLAG) once after a wait on a peer's flag ran out."""
        st = ctypes.c_uint(0)
        return self._lib.qfb_comm_read_status(self._h, torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(st))

    # -- emulation helpers (tests) ---------------------------------------------------
    def next_epoch(self, row: int = 0) -> int:
        """The epoch the next reduction of `row` will use (synchronises the stream)."""
        e = ctypes.c_uint(0)
        _native.check(self._lib.qfb_comm_epoch(self._h, row, torch.cuda.current_stream(self.device).cuda_stream,
                                               ctypes.byref(e)), "qfb_comm_epoch")
        return e.value

    def write_peer_partial(self, r: int, which: int, partial: torch.Tensor, epoch: int | None = None) -> None:
        """Play peer `r`: put its fp16 partial [rows, d] into THIS rank's receive region of slot `which`
        as the peer's reduction kernel would, every 4 data bytes followed by the epoch.  `epoch` None:
        the epoch the next reduction will use (rows of one call share it)."""
        rows = partial.shape[0]
        if epoch is None:
            epoch = self.next_epoch(0)
        ptr = self._lib.qfb_comm_region(self._h, which, r)
        words = torch.as_tensor(_DevView(ptr, (self.slot_rows, 2 * self.d), self), device=self.device).view(torch.int32)
        data = partial.contiguous().view(torch.int32)                      # [rows, d / 2]
        epoch &= 0xFFFFFFFF
        if epoch >= 1 << 31:
            epoch -= 1 << 32                                              # the same 32 bits as a signed word
        packed = torch.stack((data, torch.full_like(data, epoch)), dim=-1).reshape(rows, self.d)
        words[:rows].copy_(packed)

    def peer_words(self, r: int, which: int, source: int, rows: int) -> torch.Tensor:
        """Emulation only: the {data, epoch} words [rows, d] (int32: data words at even positions, epochs
        at odd ones) that rank `source` has stored into ITS receive region of slot `which` in rank `r`'s buffer."""
        bases = getattr(self, "_emulated", None)
        assert bases, "peer buffers are only addressable in the one-GPU emulation"
        off = self._lib.qfb_comm_region(self._h, which, source) - self.bases[self.rank]
        t = torch.as_tensor(_DevView(bases[r] + off, (self.slot_rows, 2 * self.d), self), device=self.device)
        return t.view(torch.int32)[:rows]

    def close(self):
        L = self._lib
        if self._h:
            L.qfb_comm_destroy(self._h)
            self._h = None
        with torch.cuda.device(self.device):
            for p in self._opened:
                L.qfb_comm_close(p)
            self._opened = []
            if self._owned:
                L.qfb_comm_free(self._owned)
                self._owned = None
            for p in getattr(self, "_emulated", []):
                L.qfb_comm_free(p)
            self._emulated = []
