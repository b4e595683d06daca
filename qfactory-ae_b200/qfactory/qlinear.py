"""Module API of the quantized linear layer: `QLinear.init / QLinear.empty` return an
`nn.Module` whose `forward(x)` computes `x @ dequant(W)^T` in fp16.

Same names, arguments and error behaviour as the reference (reference:
qfactory/qlinear.py:5-145).  Differences, all on purpose:
  * the packed tensors `.w/.s/.z` use the layouts of `convert.py`: `layout='tile'` (every bit
    width), `layout='fragment'` (K % 128 == 0: the tensor-core fragment order)
    or `layout='auto'` (the default: fragment whenever the shape allows it); `state_dict()` carries
    the layout, and loading packed tensors of the other layout raises;
  * the batch size is a run-time property of `forward`, not a compile-time constant, and
    `x` may have any number of leading dimensions;
  * kernel selection is a static heuristic inside the native library, so `compile_flags`
    and `base_impl` are accepted and ignored;
  * `QLinear.from_float` builds a layer from an fp16 weight.
The forward pass calls the native library through its C ABI; without it the module raises.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native, layout
from .convert import convert_params
from .quantize import asymmetric_quant


class _PackedLinear(torch.nn.Module):
    """Shared implementation: owns the packed buffers, the split-K workspace and the
    `qfb_layer` descriptor handed to the C ABI."""

    def __init__(self, in_features, out_features, n_bits, group_size, w, s, z, max_batch=16,
                 packed_layout=layout.LAYOUT_TILE):
        super().__init__()
        self.packed_layout = packed_layout
        self.in_features, self.out_features = in_features, out_features
        self.n_bits, self.group_size = n_bits, group_size
        # buffers: they follow .to()/.cuda() and are saved by state_dict()
        self.register_buffer("w", w)
        self.register_buffer("s", s)
        self.register_buffer("z", z)
        self.flags = 0
        self._desc = None
        self._ws = None
        self._ws_bytes = 0
        self._max_batch = max_batch
        self._host = None

    # -- native plumbing ---------------------------------------------------
    @property
    def _ws(self):
        return self._ws_tensor

    @_ws.setter
    def _ws(self, t):
        # the workspace pointer handed to the hot call follows the tensor
        self._ws_tensor = t
        self._ws_ptr = t.data_ptr() if t is not None else None

    def _prepare(self):
        if not self.w.is_cuda:
            raise _native.NativeError("the quantized linear layer runs on CUDA only (no CPU path); move it with .to('cuda')")
        L = _native.lib()
        d = _native.QfbLayer()
        d.qweight = self.w.data_ptr()
        d.scales = self.s.data_ptr() if self.s is not None else None
        d.zeros = self.z.data_ptr() if self.z is not None else None
        d.n, d.k, d.bits, d.group_size = self.out_features, self.in_features, self.n_bits, self.group_size
        d.layout = self.packed_layout
        nbytes = L.qfb_workspace_bytes(self._max_batch, self.out_features, self.in_features, self.n_bits)
        self._ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=self.w.device)
        self._ws_bytes = nbytes
        self._desc = d
        self._lib = L
        # pre-resolved pieces of the hot call
        self._desc_ref = ctypes.byref(d)
        self._fwd = L.qfb_linear_forward

    # -- the packed layout travels with the checkpoint ------------------------
    def get_extra_state(self):
        """[packed layout, library version]: the same bytes mean different codes under the two
        layouts, so a checkpoint must say which one it holds."""
        return torch.tensor([int(self.packed_layout), int(_native.version_or_zero())], dtype=torch.int32)

    def set_extra_state(self, state):
        saved = int(state[0])
        if saved != int(self.packed_layout):
            names = {layout.LAYOUT_TILE: "tile", layout.LAYOUT_FRAGMENT: "fragment"}
            raise RuntimeError(
                f"packed-layout mismatch: the checkpoint holds the {names.get(saved, saved)} layout, this module "
                f"expects {names.get(self.packed_layout, self.packed_layout)}; build the module with "
                f"layout={names.get(saved, saved)!r} or repack the tensors (convert.unpack_params / convert_params)")

    def _apply(self, fn, *a, **kw):
        r = super()._apply(fn, *a, **kw)
        self._desc = None  # device pointers changed
        self._host = None
        return r

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if self._desc is None:
            self._prepare()
        K, N = self.in_features, self.out_features
        assert x.dtype == torch.float16, "activations must be fp16"
        assert x.shape[-1] == K
        if x.dim() == 2 and x.is_contiguous():   # the common case: no reshape, no view of the result
            x2, lead = x, None
        else:
            lead = x.shape[:-1]
            x2 = x.reshape(-1, K)
            if not x2.is_contiguous():
                x2 = x2.contiguous()
        M = x2.shape[0]
        dev = x.device
        if out is None:
            out = torch.empty(M, N, dtype=torch.float16, device=dev)
        else:
            assert out.dtype == torch.float16 and out.is_contiguous() and out.numel() == M * N
        if dev != self.w.device:
            raise _native.NativeError(f"activations on {dev}, packed weights on {self.w.device}")
        if dev.index == torch.cuda.current_device():
            st = self._fwd(self._desc_ref, x2.data_ptr(), M, out.data_ptr(), self._ws_ptr, self._ws_bytes, self.flags,
                           torch.cuda.current_stream(dev).cuda_stream)
        else:  # the launch goes to the current device: make it the tensors' device
            with torch.cuda.device(dev):
                st = self._fwd(self._desc_ref, x2.data_ptr(), M, out.data_ptr(), self._ws_ptr, self._ws_bytes, self.flags,
                               torch.cuda.current_stream(dev).cuda_stream)
        if st != 0:
            _native.check(st, "qfb_linear_forward")
        return out if lead is None else out.view(*lead, N)

    def forward_addnorm(self, x, residual, norm_weight, eps=1e-5, x_out=None, out=None):
        """y = (rmsnorm(x + residual) * norm_weight) @ dequant(W)^T in ONE kernel (reference: the add, the norm
        and the linear are separate kernels, third_party/vllm-bitblas/vllm/model_executor/models/llama.py:260-285).
        `x` [rows, in_features] fp16, `residual` the same shape or None; the sum is written to `x_out` (a
        buffer other than `x` and `residual`, or None).  Returns y, or None where the fused kernel does not
        serve the layer or the batch (the caller then runs the three steps)."""
        if self._desc is None:
            self._prepare()
        rows = x.shape[0]
        if not (self.packed_layout == layout.LAYOUT_FRAGMENT and self.n_bits == 4 and self.group_size != 64 and 0 < rows <= 16
                and x.dim() == 2 and x.is_contiguous()):
            return None
        if out is None:
            out = torch.empty(rows, self.out_features, dtype=torch.float16, device=x.device)
        with torch.cuda.device(x.device):
            st = self._lib.qfb_linear_addnorm_forward(
                self._desc_ref, x.data_ptr(), None if residual is None else residual.data_ptr(),
                None if x_out is None else x_out.data_ptr(), norm_weight.data_ptr(), float(eps), rows, out.data_ptr(),
                self._ws_ptr, self._ws_bytes, self.flags, torch.cuda.current_stream(x.device).cuda_stream)
        if st == 3:    # QFB_ERR_UNSUPPORTED
            return None
        if st != 0:
            _native.check(st, "qfb_linear_addnorm_forward")
        return out

    def silu_mul_supported(self, rows: int) -> bool:
        """True when `forward_silu_mul` runs as ONE kernel for `rows` activation rows."""
        return self.packed_layout == layout.LAYOUT_FRAGMENT and 0 < rows <= (8 if self.n_bits == 3 else 16)

    def forward_silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """(silu(gate) * up) @ dequant(W)^T for gate_up [..., 2 * in_features] = [gate | up], the down
        projection of a gated MLP with its activation fused in (reference:
        third_party/vllm-bitblas/vllm/model_executor/models/llama.py:91-96 runs the activation as a
        launch of its own).  One kernel on fragment-layout layers up to 16 rows; otherwise the
        element-wise kernel followed by `forward`.  Both give the same bits."""
        if self._desc is None:
            self._prepare()
        assert gate_up.dtype == torch.float16 and gate_up.shape[-1] == 2 * self.in_features
        g2 = gate_up.reshape(-1, 2 * self.in_features)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        M = g2.shape[0]
        if not self.silu_mul_supported(M):
            from . import ops

            return self.forward(ops.silu_mul(g2), out=out)
        if out is None:
            out = torch.empty(M, self.out_features, dtype=torch.float16, device=g2.device)
        else:
            assert out.dtype == torch.float16 and out.is_contiguous() and out.numel() == M * self.out_features
        with torch.cuda.device(g2.device):
            st = self._lib.qfb_linear_silu_mul_forward(
                ctypes.byref(self._desc), g2.data_ptr(), M, out.data_ptr(), self._ws.data_ptr(), self._ws_bytes, self.flags,
                torch.cuda.current_stream(g2.device).cuda_stream)
        if st != 0:
            _native.check(st, "qfb_linear_silu_mul_forward")
        return out.view(*gate_up.shape[:-1], self.out_features)

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor | None = None, sync: bool = True) -> torch.Tensor:
        """Host-buffer entry: `x_host` (CPU fp16, ideally pinned) is copied in, the result is
        copied back into `y_host` (CPU fp16) and the stream is synchronised.  With `sync=False` the
        call only queues the work: `y_host` is valid after the caller has synchronised the stream
        (several layers can be queued and waited for once)."""
        if self._desc is None:
            self._prepare()
        x2 = x_host.reshape(-1, self.in_features)
        M = x2.shape[0]
        assert x2.dtype == torch.float16 and x2.is_contiguous() and not x2.is_cuda
        if y_host is None:
            y_host = torch.empty(M, self.out_features, dtype=torch.float16, pin_memory=True)
        if self._host is None or self._host[0].shape[0] < M:
            dev = self.w.device
            self._host = (torch.empty(M, self.in_features, dtype=torch.float16, device=dev),
                          torch.empty(M, self.out_features, dtype=torch.float16, device=dev))
        xs, ys = self._host
        st = self._lib.qfb_linear_forward_host(
            ctypes.byref(self._desc), x2.data_ptr(), M, y_host.data_ptr(), xs.data_ptr(), ys.data_ptr(),
            self._ws.data_ptr(), self._ws_bytes, self.flags | (0 if sync else _native.FLAG_NO_SYNC),
            torch.cuda.current_stream(self.w.device).cuda_stream,
        )
        if st != 0:
            _native.check(st, "qfb_linear_forward_host")
        return y_host

    def unpack_torch(self):
        """(codes int32 [K,N], scales fp16 [K/GS,N] or None, effective zeros int32 [K/GS,N] or None)
        recovered from the packed buffers in torch, on whatever device they live on."""
        N, K = self.out_features, self.in_features
        if self.packed_layout == layout.LAYOUT_FRAGMENT:
            return (layout.unpack_weight_fragment(self.w, N, K, self.n_bits),
                    layout.unpack_scale_fragment(self.s, N) if self.s is not None else None,
                    layout.unpack_zero_fragment(self.z, N) if self.z is not None else None)
        return (layout.unpack_weight(self.w, N, K, self.n_bits),
                layout.unpack_scale(self.s, N) if self.s is not None else None,
                layout.unpack_zero(self.z, N) if self.z is not None else None)

    # -- test / debug helpers through the kernels' own decode path ----------
    def unpack_codes(self) -> torch.Tensor:
        if self._desc is None:
            self._prepare()
        q = torch.empty(self.in_features, self.out_features, dtype=torch.int32, device=self.w.device)
        _native.check(self._lib.qfb_unpack_codes(ctypes.byref(self._desc), q.data_ptr(),
                                                 torch.cuda.current_stream(self.w.device).cuda_stream))
        return q

    def dequantize(self) -> torch.Tensor:
        if self._desc is None:
            self._prepare()
        wd = torch.empty(self.in_features, self.out_features, dtype=torch.float16, device=self.w.device)
        _native.check(self._lib.qfb_dequantize(ctypes.byref(self._desc), wd.data_ptr(),
                                               torch.cuda.current_stream(self.w.device).cuda_stream))
        return wd

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.n_bits}, "
                f"group_size={self.group_size}, symmetric={self.z is None and self.s is not None}, "
                f"layout={'fragment' if self.packed_layout else 'tile'}")


class GPTQLinear(_PackedLinear):
    """Group-quantized layer (reference: qfactory/qlinear.py:5-58)."""

    def __init__(self, in_features, out_features, n_bits, weight, group_size, scale, zero, bias,
                 compile_flags=None, skip_convert=False, batch_size=1, base_impl=False, layout_kind="auto"):
        if bias:
            raise NotImplementedError("Bias is not supported")
        lay = layout.resolve_layout(layout_kind, out_features, in_features, n_bits, group_size, batch_size)
        if skip_convert:
            w, s, z = weight, scale, zero
        else:
            w, s, z = convert_params(
                {"K": in_features, "N": out_features, "NBITS": n_bits, "GS": group_size, "LAYOUT": lay},
                (weight, scale, zero))
        npad = layout.padded_rows(out_features)
        layout.check_shape(out_features, in_features, n_bits, group_size)
        assert w.dtype == torch.int8 and w.dim() == 2
        assert w.numel() == npad * in_features * n_bits // 8
        assert s.dtype == torch.float16 and s.shape == (npad, in_features // group_size)
        if z is not None:
            assert z.dtype == torch.int8 and z.shape == (npad, in_features // group_size)
        super().__init__(in_features, out_features, n_bits, group_size, w, s, z, max_batch=max(16, batch_size),
                         packed_layout=lay)


class GEMVLinear(_PackedLinear):
    """Group-less layer on raw unsigned codes: y = x @ codes^T, no scale or zero
    (reference: qfactory/qlinear.py:60-97, kernel qfactory/include/gemv.h:12-94)."""

    def __init__(self, in_features, out_features, n_bits, weight, bias, compile_flags=None, skip_convert=False,
                 batch_size=1, layout_kind="auto"):
        if bias:
            raise NotImplementedError("Bias is not supported")
        lay = layout.resolve_layout(layout_kind, out_features, in_features, n_bits, -1, batch_size)
        w = weight if skip_convert else convert_params(
            {"K": in_features, "N": out_features, "NBITS": n_bits, "LAYOUT": lay}, (weight,))
        layout.check_shape(out_features, in_features, n_bits, -1)
        assert w.dtype == torch.int8 and w.dim() == 2
        assert w.numel() == layout.padded_rows(out_features) * in_features * n_bits // 8
        super().__init__(in_features, out_features, n_bits, -1, w, None, None, max_batch=max(16, batch_size),
                         packed_layout=lay)


class QLinear:
    """Factory with the reference's static methods (reference: qfactory/qlinear.py:99-145)."""

    @staticmethod
    def init(batch_size, in_features, out_features, n_bits, weight, group_size=-1, scale=None, zero=None,
             bias=False, compile_flags={}, layout="auto"):
        if group_size == -1:
            return GEMVLinear(in_features, out_features, n_bits, weight, bias, compile_flags, skip_convert=False,
                              batch_size=batch_size, layout_kind=layout)
        return GPTQLinear(in_features, out_features, n_bits, weight, group_size, scale, zero, bias, compile_flags,
                          skip_convert=False, batch_size=batch_size, layout_kind=layout)

    @staticmethod
    def empty(M, K, N, NBITS, GS, sym, compile_flags={}, base_impl=False, device="cuda", layout="auto"):
        """Uninitialised packed buffers of the right shapes (benchmarks, the vLLM hook)."""
        from . import layout as _layout
        npad = _layout.padded_rows(N)
        w = torch.empty(npad, K * NBITS // 8, dtype=torch.int8, device=device)
        if GS == -1:
            return GEMVLinear(K, N, NBITS, w, False, compile_flags, skip_convert=True, batch_size=M, layout_kind=layout)
        s = torch.empty(npad, K // GS, dtype=torch.float16, device=device)
        z = None if sym else torch.empty(npad, K // GS, dtype=torch.int8, device=device)
        return GPTQLinear(K, N, NBITS, w, GS, s, z, False, compile_flags, skip_convert=True, batch_size=M,
                          base_impl=base_impl, layout_kind=layout)

    @staticmethod
    def from_float(weight: torch.Tensor, n_bits: int, group_size: int = 128, batch_size: int = 1, layout="auto"):
        """Quantize an fp16 weight [K, N] group-wise (asymmetric, as the reference's
        tests/acc_gptq.py:10-29 does) and pack it."""
        K, N = weight.shape
        q, s, z = asymmetric_quant(weight, group_size, n_bits)
        return QLinear.init(batch_size, K, N, n_bits, q, group_size, s, z, layout=layout)
