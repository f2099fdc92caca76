"""``Sm100Backend``: the reference's ``Backend`` linear family (crates/velox-core/src/backend.rs
:897-1141) served by the sm_100a kernels through the C ABI of include/velox_sm100.h.

Device memory is held in torch tensors (plumbing only): f32 buffers are ``torch.float32``, bf16
twins ``torch.bfloat16``, encoded weights ``torch.uint8``. Every call validates its arguments as
the reference's ``check::linear`` does, then makes exactly one FFI call; work is queued on torch's
current CUDA stream and nothing is synchronised. There is no CPU path."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .errors import ShapeError, Unsupported, status
from .weights import (ActPolicy, ActQuant, LinearDst, WeightFormat, WeightView, align256,
                      check_linear, check_weight)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dev(t: torch.Tensor, dtype, what: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ShapeError(f"{what}: expected a CUDA tensor")
    if t.dtype != dtype or not t.is_contiguous():
        raise ShapeError(f"{what}: expected contiguous {dtype}, got {t.dtype}")
    return t


def _view_struct(w: WeightView) -> _lib.View:
    return _lib.View(w.buf.data_ptr(), int(w.format), w.act.kind, w.parent_rows, w.k, w.row_begin,
                     w.rows, w.act.divisor)


class Sm100Backend:
    """One CUDA device. Mirrors ``CudaBackend`` + ``CudaKernels`` for the linear family
    (crates/velox-cuda/src/lib.rs:550-760, 1840-1882, 2084-2128, 2931-2950)."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("Sm100Backend needs a CUDA device (no CPU fallback)")
        self.device = torch.device("cuda", device)
        self.lib = _lib.lib()
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise RuntimeError(f"built for sm_100a only; device is sm_{major}{minor}")

    # ---- buffers (Backend::alloc / upload / upload_bytes / download, backend.rs:907-918) ----
    def alloc(self, n: int) -> torch.Tensor:
        return torch.zeros(n, dtype=torch.float32, device=self.device)

    def upload(self, data) -> torch.Tensor:
        return torch.as_tensor(data, dtype=torch.float32).contiguous().to(self.device)

    def upload_bytes(self, data) -> torch.Tensor:
        """Raw payload bytes, zero-padded to a 4-byte slot (crates/velox-cuda/src/lib.rs:1746-1757)."""
        t = torch.as_tensor(data, dtype=torch.uint8).reshape(-1)
        pad = (-t.numel()) % 4
        if pad:
            t = torch.cat([t, torch.zeros(pad, dtype=torch.uint8)])
        return t.contiguous().to(self.device)

    def download(self, buf: torch.Tensor) -> torch.Tensor:
        return buf.detach().cpu()

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def _bind(self) -> None:
        torch.cuda.set_device(self.device)
        self.lib.velox_sm100_set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    # ---- linear family --------------------------------------------------------------------
    def linear_act(self, w: WeightView, m: int) -> ActQuant:
        """Backend::linear_act (backend.rs:933-937)."""
        check_weight(w, w.buf.numel())
        div = C.c_float(0.0)
        code = self.lib.velox_sm100_linear_act(C.byref(_view_struct(w)), m, C.byref(div))
        if code < 0:
            status(code, "linear_act")
        return ActQuant(code, div.value)

    def takes_bf16(self, w: WeightView, m: int) -> bool:
        """Backend::takes_bf16 (backend.rs:1005-1010)."""
        return self.linear_act(w, m).kind == ActQuant.BF16

    def bf16_twins(self) -> bool:
        return True

    def linear(self, x: torch.Tensor, w: WeightView, y: torch.Tensor, m: int,
               yb: Optional[torch.Tensor] = None) -> None:
        """Backend::linear (backend.rs:925-932): y[m, rows] = x[m, k] . W^T."""
        _dev(x, torch.float32, "linear x"); _dev(y, torch.float32, "linear y")
        _dev(w.buf, torch.uint8, "linear w")
        check_linear(x.numel(), w, w.buf.numel(), y.numel(), m)
        if yb is not None:
            _dev(yb, torch.bfloat16, "linear yb")
        self._bind()
        status(self.lib.velox_sm100_linear_view(x.data_ptr(), C.byref(_view_struct(w)), m,
                                                y.data_ptr(), _ptr(yb)), "sm100 linear")

    def linear_bf16(self, xb: torch.Tensor, w: WeightView, y: Optional[torch.Tensor], m: int,
                    yb: Optional[torch.Tensor] = None) -> None:
        """Backend::linear_bf16 (backend.rs:1011-1021)."""
        _dev(xb, torch.bfloat16, "linear_bf16 xb")
        _dev(w.buf, torch.uint8, "linear_bf16 w")
        out_len = y.numel() if y is not None else yb.numel()
        check_linear(xb.numel(), w, w.buf.numel(), out_len, m)
        self._bind()
        status(self.lib.velox_sm100_linear_bf16(xb.data_ptr(), C.byref(_view_struct(w)), m,
                                                _ptr(y), _ptr(yb)), "sm100 linear_bf16")

    def linear_swiglu_act(self, gate: WeightView, up: WeightView, m: int) -> ActQuant:
        div = C.c_float(0.0)
        code = self.lib.velox_sm100_linear_swiglu_act(C.byref(_view_struct(gate)),
                                                      C.byref(_view_struct(up)), m, C.byref(div))
        if code < 0:
            status(code, "linear_swiglu_act")
        return ActQuant(code, div.value)

    def fuses_swiglu(self, gate: WeightView, up: WeightView, m: int) -> bool:
        return True

    def swiglu_twin(self, gate: WeightView, up: WeightView, m: int) -> bool:
        return self.linear_swiglu_act(gate, up, m).kind == ActQuant.BF16

    def _check_swiglu(self, x_len, gate, up, out_len, m):
        check_linear(x_len, gate, gate.buf.numel(), out_len, m)
        check_linear(x_len, up, up.buf.numel(), out_len, m)
        if up.rows != gate.rows or up.k != gate.k:
            raise ShapeError(f"linear_swiglu: gate [{gate.rows},{gate.k}] and up [{up.rows},{up.k}] differ")

    def linear_swiglu(self, x: torch.Tensor, gate: WeightView, up: WeightView, out: torch.Tensor,
                      m: int, scratch: Optional[torch.Tensor] = None,
                      outb: Optional[torch.Tensor] = None) -> None:
        """Backend::linear_swiglu (backend.rs:1102-1118), always fused: ``scratch`` is unused."""
        _dev(x, torch.float32, "linear_swiglu x"); _dev(out, torch.float32, "linear_swiglu out")
        self._check_swiglu(x.numel(), gate, up, out.numel(), m)
        self._bind()
        status(self.lib.velox_sm100_linear_swiglu(x.data_ptr(), C.byref(_view_struct(gate)),
                                                  C.byref(_view_struct(up)), m, out.data_ptr(),
                                                  _ptr(outb)), "sm100 linear_swiglu")

    def linear_swiglu_twin(self, xb: torch.Tensor, gate: WeightView, up: WeightView,
                           out: Optional[torch.Tensor], outb: Optional[torch.Tensor], m: int) -> None:
        """Backend::linear_swiglu_twin (backend.rs:1034-1048)."""
        _dev(xb, torch.bfloat16, "linear_swiglu_twin xb")
        out_len = out.numel() if out is not None else outb.numel()
        self._check_swiglu(xb.numel(), gate, up, out_len, m)
        self._bind()
        status(self.lib.velox_sm100_linear_swiglu_bf16(xb.data_ptr(), C.byref(_view_struct(gate)),
                                                       C.byref(_view_struct(up)), m, _ptr(out),
                                                       _ptr(outb)), "sm100 linear_swiglu_twin")

    def linears(self, x: Optional[torch.Tensor], xb: Optional[torch.Tensor],
                dsts: Sequence[LinearDst], m: int) -> None:
        """Backend::linears (backend.rs:938-958): parts into column ranges, no scratch."""
        parts = []
        x_len = x.numel() if x is not None else xb.numel()
        for d in dsts:
            _dev(d.y, torch.float32, "linears y")
            for p in d.parts:
                check_linear(x_len, p.w, p.w.buf.numel(), d.y.numel(), m)
                if p.col + p.w.rows > d.ld or d.y.numel() < m * d.ld:
                    raise ShapeError(f"linears: columns {p.col}..{p.col + p.w.rows} of {m} x {d.ld} "
                                     f"in {d.y.numel()} values")
                parts.append(_lib.Part(_view_struct(p.w), d.y.data_ptr(), d.ld, p.col))
        arr = (_lib.Part * len(parts))(*parts)
        self._bind()
        status(self.lib.velox_sm100_linears(_ptr(x), _ptr(xb), arr, len(parts), m), "sm100 linears")

    def matmul(self, x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, n: int, k: int) -> None:
        """Backend::matmul (backend.rs:1550-1564): y[m, n] = x[m, k] . w[n, k]^T, f32."""
        _dev(x, torch.float32, "matmul x"); _dev(w, torch.float32, "matmul w"); _dev(y, torch.float32, "matmul y")
        if m <= 0 or n <= 0 or k <= 0 or x.numel() < m * k or w.numel() < n * k or y.numel() < m * n:
            raise ShapeError(f"matmul [{m},{k}] x [{n},{k}]^T -> [{m},{n}]: buffers {x.numel()}, {w.numel()}, {y.numel()}")
        self._bind()
        status(self.lib.velox_sm100_matmul(x.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k), "sm100 matmul")

    def embed_from(self, ids: torch.Tensor, offset: int, count: int, table: WeightView, out: torch.Tensor) -> None:
        """Backend::embed_from (backend.rs:1149-1160): rows ``ids[offset : offset + count]`` of the table
        view, decoded exactly; ``ids`` is a device int32 tensor."""
        _dev(out, torch.float32, "embed out")
        if ids.dtype != torch.int32 or not ids.is_cuda:
            raise ShapeError("embed ids: expected a CUDA int32 tensor")
        check_weight(table, table.buf.numel())
        if offset < 0 or count < 0 or offset + count > ids.numel() or out.numel() < count * table.k:
            raise ShapeError(f"embed: ids {offset}+{count} of {ids.numel()}, out {out.numel()} for {count} x {table.k}")
        self._bind()
        status(self.lib.velox_sm100_embed(ids.data_ptr() + 4 * offset, count, table.buf.data_ptr(), int(table.format),
                                          table.parent_rows, table.k, table.row_begin, out.data_ptr()), "sm100 embed")

    def embed(self, ids, table: WeightView, out: torch.Tensor) -> None:
        """Backend::embed (backend.rs:1142-1148): host ids, each checked against the view's rows."""
        ids = [int(i) for i in ids]
        if any(i < 0 or i >= table.rows for i in ids):
            raise ShapeError(f"embed: id outside the table's {table.rows} rows")
        if not ids:
            return
        dev_ids = torch.tensor(ids, dtype=torch.int32, device=self.device)
        self.embed_from(dev_ids, 0, len(ids), table, out)

    # ---- neighbours --------------------------------------------------------------------------
    def dequant_rows(self, w: WeightView) -> torch.Tensor:
        """Exact decode of the view, the values format::decode_rows produces."""
        check_weight(w, w.buf.numel())
        out = torch.empty(w.rows, w.k, dtype=torch.float32, device=self.device)
        self._bind()
        status(self.lib.velox_sm100_dequant_rows(C.byref(_view_struct(w)), out.data_ptr()),
               "sm100 dequant_rows")
        return out

    def quantize_act_fp8row(self, x: torch.Tensor):
        m, k = x.shape
        codes = torch.empty(m, k, dtype=torch.uint8, device=self.device)
        scales = torch.empty(m, dtype=torch.float32, device=self.device)
        self._bind()
        status(self.lib.velox_sm100_quantize_act_fp8row(x.data_ptr(), m, k, codes.data_ptr(),
                                                        scales.data_ptr()), "quantize fp8row")
        return codes, scales

    def quantize_act_nvfp4(self, x: torch.Tensor, divisor: float):
        m, k = x.shape
        mp = (m + 127) // 128 * 128
        codes = torch.empty(m, k // 2, dtype=torch.uint8, device=self.device)
        atoms = torch.empty(mp * k // 16, dtype=torch.uint8, device=self.device)
        self._bind()
        status(self.lib.velox_sm100_quantize_act_nvfp4(x.data_ptr(), m, k, divisor, codes.data_ptr(),
                                                       atoms.data_ptr()), "quantize nvfp4")
        return codes, atoms

    def encode_nvfp4(self, w: torch.Tensor) -> torch.Tensor:
        """NVFP4 payload of an f32 [n, k] device matrix (benchmark weight construction)."""
        _dev(w, torch.float32, "encode_nvfp4 w")
        n, k = w.shape
        WeightFormat.NVFP4.check_shape(n, k)
        payload = torch.zeros(align256(WeightFormat.NVFP4.payload_bytes(n, k)), dtype=torch.uint8,
                              device=self.device)
        amax = float(w.abs().max().item())
        self._bind()
        status(self.lib.velox_sm100_encode_nvfp4(w.data_ptr(), n, k, amax, payload.data_ptr()),
               "encode_nvfp4")
        return payload

    def swiglu(self, src, rows, src_cols, gate, up, width, out) -> None:
        self._bind()
        status(self.lib.velox_sm100_swiglu(src.data_ptr(), rows, src_cols, gate, up, width,
                                           out.data_ptr()), "sm100 swiglu")

    def silu_mul(self, gate, up, n) -> None:
        self._bind()
        status(self.lib.velox_sm100_silu_mul(gate.data_ptr(), up.data_ptr(), n), "sm100 silu_mul")

    def add(self, acc, x, n) -> None:
        self._bind()
        status(self.lib.velox_sm100_add(acc.data_ptr(), x.data_ptr(), n), "sm100 add")

    def add_rms_norm_twin(self, acc, x, weight, y, yb, rows, dim, eps, offset=False, xb=None) -> None:
        """Backend::add_rms_norm_twin (backend.rs:968-983); x None = plain rms_norm of acc. With
        ``xb`` the addend is a bf16 buffer (the all-reduced partial sums of a row-split projection)."""
        self._bind()
        if xb is not None:
            status(self.lib.velox_sm100_add_bf16_rms_norm_twin(
                acc.data_ptr(), xb.data_ptr(), weight.data_ptr(), _ptr(y), _ptr(yb), rows, dim, eps,
                int(offset)), "sm100 add_bf16_rms_norm_twin")
            return
        status(self.lib.velox_sm100_add_rms_norm_twin(acc.data_ptr(), _ptr(x), weight.data_ptr(),
                                                      _ptr(y), _ptr(yb), rows, dim, eps,
                                                      int(offset)), "sm100 add_rms_norm_twin")

    # -- FP4 activation twins (the NVFP4 counterpart of add_rms_norm_q8 / linear_q8 /
    #    linear_swiglu_q8, crates/velox-core/src/backend.rs:1050-1100)
    def q4_blob(self, rows: int, dim: int):
        """Device storage for [rows, dim] NVFP4 activations: (codes, atoms)."""
        codes = torch.zeros(rows * dim // 2, dtype=torch.uint8, device=self.device)
        atoms = torch.zeros((rows + 127) // 128 * 128 * dim // 16, dtype=torch.uint8, device=self.device)
        return codes, atoms

    def add_rms_norm_q4(self, acc, x, weight, yb, q4, rows, dim, eps, divisor, offset=False, xb=None) -> None:
        self._bind()
        status(self.lib.velox_sm100_add_rms_norm_q4(acc.data_ptr(), _ptr(x), _ptr(xb), weight.data_ptr(),
                                                    _ptr(yb), q4[0].data_ptr(), q4[1].data_ptr(), rows, dim,
                                                    eps, 1 if offset else 0, divisor), "sm100 add_rms_norm_q4")

    def linear_q4(self, q4, divisor: float, w: WeightView, y: Optional[torch.Tensor], m: int,
                  yb: Optional[torch.Tensor] = None) -> None:
        self._bind()
        status(self.lib.velox_sm100_linear_q4(q4[0].data_ptr(), q4[1].data_ptr(), divisor,
                                              C.byref(_view_struct(w)), m, _ptr(y), _ptr(yb)), "sm100 linear_q4")

    def linear_swiglu_q4(self, q4, divisor: float, gate: WeightView, up: WeightView,
                         out: Optional[torch.Tensor], outb: Optional[torch.Tensor], m: int) -> None:
        self._bind()
        status(self.lib.velox_sm100_linear_swiglu_q4(q4[0].data_ptr(), q4[1].data_ptr(), divisor,
                                                     C.byref(_view_struct(gate)), C.byref(_view_struct(up)), m,
                                                     _ptr(out), _ptr(outb)), "sm100 linear_swiglu_q4")

    def linear_q4_to_q4(self, q4, divisor: float, w: WeightView, m: int, out_q4, out_divisor: float,
                        yb: Optional[torch.Tensor] = None) -> None:
        """linear_q4 whose result is (also) the next linear's NVFP4 input."""
        self._bind()
        status(self.lib.velox_sm100_linear_q4_to_q4(q4[0].data_ptr(), q4[1].data_ptr(), divisor,
                                                    C.byref(_view_struct(w)), m, _ptr(yb), out_q4[0].data_ptr(),
                                                    out_q4[1].data_ptr(), out_divisor), "sm100 linear_q4_to_q4")

    def linear_swiglu_q4_to_q4(self, q4, divisor: float, gate: WeightView, up: WeightView, m: int, out_q4,
                               out_divisor: float, outb: Optional[torch.Tensor] = None) -> None:
        self._bind()
        status(self.lib.velox_sm100_linear_swiglu_q4_to_q4(
            q4[0].data_ptr(), q4[1].data_ptr(), divisor, C.byref(_view_struct(gate)), C.byref(_view_struct(up)), m,
            _ptr(outb), out_q4[0].data_ptr(), out_q4[1].data_ptr(), out_divisor), "sm100 linear_swiglu_q4_to_q4")

    @staticmethod
    def _parts_q4(parts):
        arr = (_lib.PartQ4 * len(parts))()
        for i, (w, yb, oq, od) in enumerate(parts):
            arr[i] = _lib.PartQ4(_view_struct(w), _ptr(yb), None if oq is None else oq[0].data_ptr(),
                                 None if oq is None else oq[1].data_ptr(), od)
        return arr

    def linears_q4(self, q4, divisor: float, parts, m: int) -> None:
        """parts: (view, yb or None, out_q4 or None, out_divisor) per projection of the same input."""
        self._bind()
        arr = self._parts_q4(parts)
        status(self.lib.velox_sm100_linears_q4(q4[0].data_ptr(), q4[1].data_ptr(), divisor, arr, len(parts), m),
               "sm100 linears_q4")

    # -- tensor parallelism: reduce-scatter fused into the row-split linear, all-gather into the norm;
    #    `sync` (a _lib.TpSync or None) names the peers' flags a launch waits for and raises
    @staticmethod
    def _sync(sync):
        return None if sync is None else C.byref(sync)

    def tp_make_maps(self, maps_dev: torch.Tensor, slot_ptrs, rows_per_owner: int, cols: int) -> None:
        self._bind()
        arr = (C.c_uint64 * len(slot_ptrs))(*slot_ptrs)
        status(self.lib.velox_sm100_tp_make_maps(maps_dev.data_ptr(), arr, len(slot_ptrs), rows_per_owner, cols),
               "sm100 tp_make_maps")

    def tp_step_begin(self, epoch: torch.Tensor) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_step_begin(epoch.data_ptr()), "sm100 tp_step_begin")

    def tp_wait(self, sync) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_wait(C.byref(sync)), "sm100 tp_wait")

    def tp_barrier(self, sync) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_barrier(C.byref(sync)), "sm100 tp_barrier")

    def tp_signal(self, sync) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_signal(C.byref(sync)), "sm100 tp_signal")

    def tp_linears_q4(self, q4, divisor: float, parts, m: int, sync=None) -> None:
        self._bind()
        arr = self._parts_q4(parts)
        status(self.lib.velox_sm100_tp_linears_q4(q4[0].data_ptr(), q4[1].data_ptr(), divisor, arr, len(parts), m,
                                                  self._sync(sync)), "sm100 tp_linears_q4")

    def tp_linear_swiglu_q4_to_q4(self, q4, divisor: float, gate: WeightView, up: WeightView, m: int, out_q4,
                                  out_divisor: float, outb: Optional[torch.Tensor] = None, sync=None) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_linear_swiglu_q4_to_q4(
            q4[0].data_ptr(), q4[1].data_ptr(), divisor, C.byref(_view_struct(gate)), C.byref(_view_struct(up)), m,
            _ptr(outb), out_q4[0].data_ptr(), out_q4[1].data_ptr(), out_divisor, self._sync(sync)),
            "sm100 tp_linear_swiglu_q4_to_q4")

    def tp_linear_q4_scatter(self, q4, divisor: float, w: WeightView, m: int, maps_dev: torch.Tensor,
                             rows_per_owner: int, sync=None) -> None:
        self._bind()
        status(self.lib.velox_sm100_tp_linear_q4_scatter(q4[0].data_ptr(), q4[1].data_ptr(), divisor,
                                                         C.byref(_view_struct(w)), m, maps_dev.data_ptr(),
                                                         rows_per_owner, self._sync(sync)), "sm100 tp_linear_q4_scatter")

    def tp_norm_q4(self, acc, slots, nslots: int, slot_stride: int, weight, codes_ptrs, atoms_ptrs, row0: int,
                   rows: int, dim: int, eps: float, divisor: float, offset=False, sync=None) -> None:
        self._bind()
        n = len(codes_ptrs)
        status(self.lib.velox_sm100_tp_norm_q4(acc.data_ptr(), _ptr(slots), nslots, slot_stride, weight.data_ptr(),
                                               (C.c_uint64 * n)(*codes_ptrs), (C.c_uint64 * n)(*atoms_ptrs), n, row0,
                                               rows, dim, eps, 1 if offset else 0, divisor, self._sync(sync)),
               "sm100 tp_norm_q4")

    def tp_finish(self, acc, slots, nslots: int, slot_stride: int, out_ptrs, row0: int, rows: int, dim: int,
                  sync=None) -> None:
        self._bind()
        n = len(out_ptrs)
        status(self.lib.velox_sm100_tp_finish(acc.data_ptr(), slots.data_ptr(), nslots, slot_stride,
                                              (C.c_uint64 * n)(*out_ptrs), n, row0, rows, dim, self._sync(sync)),
               "sm100 tp_finish")

    def debug_status(self) -> int:
        return int(self.lib.velox_sm100_debug_status())

    def debug_status_reset(self) -> None:
        status(self.lib.velox_sm100_debug_status_reset(), "sm100 debug_status_reset")

    def add_bf16(self, acc, xb, n) -> None:
        self._bind()
        status(self.lib.velox_sm100_add_bf16(acc.data_ptr(), xb.data_ptr(), n), "sm100 add_bf16")

    def bf16_twin_into(self, x: torch.Tensor, xb: torch.Tensor, n: int) -> torch.Tensor:
        self._bind()
        status(self.lib.velox_sm100_bf16_twin(x.data_ptr(), xb.data_ptr(), n), "bf16_twin")
        return xb

    # ---- measurement hooks (crates/velox-cuda/src/timing.rs) ---------------------------------
    TIMED_CLASSES = ("gemv", "gemm_nvfp4", "gemm_fp8", "gemm_bf16", "act_quant", "dequant", "norm")

    def timing_enable(self, on: bool) -> None:
        self.lib.velox_sm100_timing_enable(int(on))

    def timing_collect(self) -> dict:
        """Summed kernel milliseconds and launch counts per class since the last collect."""
        n = len(self.TIMED_CLASSES)
        ms = (C.c_double * n)()
        cnt = (C.c_longlong * n)()
        status(self.lib.velox_sm100_timing_collect(ms, cnt, n), "timing_collect")
        return {name: (ms[i], cnt[i]) for i, name in enumerate(self.TIMED_CLASSES)}

    def launch_count(self) -> int:
        return int(self.lib.velox_sm100_launch_count())

    def bf16_twin(self, x: torch.Tensor) -> torch.Tensor:
        xb = torch.empty(x.shape, dtype=torch.bfloat16, device=self.device)
        self._bind()
        status(self.lib.velox_sm100_bf16_twin(x.data_ptr(), xb.data_ptr(), x.numel()), "bf16_twin")
        return xb
