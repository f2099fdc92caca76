"""Host-side types of the linear path, mirroring the reference's contract:
``WeightFormat`` (crates/velox-core/src/format.rs:12-35, 117-173), ``ActPolicy`` / ``ActQuant``
(crates/velox-core/src/backend.rs:757-806), ``WeightView`` (backend.rs:826-895), ``LinearPart`` /
``LinearDst`` (backend.rs:847-867), ``swiglu_pair`` (backend.rs:2236-2270) and the shape checks
of crates/velox-core/src/check.rs:100-131. Pure Python; no device work happens here."""
from __future__ import annotations

import enum
from dataclasses import dataclass, replace
from typing import Any, Optional, Sequence

from .errors import ShapeError, Unsupported


class WeightFormat(enum.IntEnum):
    """Stored encodings this kernel set executes; values are the launcher format codes
    (crates/velox-cuda/src/portable.rs:197-216)."""

    FP8_ROW_BF16 = 2   # fp8_e4m3fn_row_bf16 / row_scale_v1
    NVFP4 = 3          # nvfp4 / block_scale_k16_m128x4_v1
    GGML_Q4_K = 17     # ggml_q4_k / ggml_block_v1 (crates/velox-core/src/ggml.rs:51-68)

    @property
    def format_name(self) -> str:
        return {2: "fp8_e4m3fn_row_bf16", 3: "nvfp4", 17: "ggml_q4_k"}[int(self)]

    @property
    def layout(self) -> str:
        return {2: "row_scale_v1", 3: "block_scale_k16_m128x4_v1", 17: "ggml_block_v1"}[int(self)]

    @staticmethod
    def from_names(fmt: str, layout: str) -> "WeightFormat":
        table = {("fp8_e4m3fn_row_bf16", "row_scale_v1"): WeightFormat.FP8_ROW_BF16,
                 ("nvfp4", "block_scale_k16_m128x4_v1"): WeightFormat.NVFP4,
                 ("ggml_q4_k", "ggml_block_v1"): WeightFormat.GGML_Q4_K}
        try:
            return table[(fmt, layout)]
        except KeyError:
            raise Unsupported(f"weight format {fmt} / {layout}") from None

    def check_shape(self, n: int, k: int) -> None:
        """format.rs:117-145."""
        if n <= 0 or k <= 0:
            raise ShapeError(f"{self.format_name} matrix [{n},{k}] is empty")
        if self is WeightFormat.NVFP4 and (n % 128 != 0 or k % 64 != 0):
            raise ShapeError(f"nvfp4 needs N % 128 == 0 and K % 64 == 0, got [{n},{k}]")
        if self is WeightFormat.GGML_Q4_K and k % 256 != 0:
            raise ShapeError(f"q4_k needs K % 256 == 0, got [{n},{k}]")

    def payload_bytes(self, n: int, k: int) -> int:
        """format.rs:147-160."""
        if self is WeightFormat.FP8_ROW_BF16:
            return align256(n * k) + 2 * n
        if self is WeightFormat.NVFP4:
            return align256(n * k // 2) + n * k // 16 + 4
        return n * (k // 256) * 144


def align256(x: int) -> int:
    return (x + 255) // 256 * 256


def nvfp4_scale_offset(n: int, g: int, k: int) -> int:
    """format.rs:345-354."""
    k_tiles = k // 64
    row_tile, row_inner = divmod(n, 128)
    return (row_tile * k_tiles + g // 4) * 512 + (row_inner % 32) * 16 + (row_inner // 32) * 4 + g % 4


@dataclass(frozen=True)
class ActPolicy:
    """backend.rs:757-780. kind: 0 A16Only, 1 AllowA8, 2 AllowA4{divisor}."""

    kind: int = 0
    divisor: float = 0.0

    @staticmethod
    def a16_only() -> "ActPolicy":
        return ActPolicy(0)

    @staticmethod
    def allow_a8() -> "ActPolicy":
        return ActPolicy(1)

    @staticmethod
    def allow_a4(divisor: float) -> "ActPolicy":
        return ActPolicy(2, float(divisor))

    def meet(self, other: "ActPolicy") -> "ActPolicy":
        if self.kind == 0 or other.kind == 0:
            return ActPolicy(0)
        if self.kind == 2 and other.kind == 2 and self.divisor == other.divisor:
            return self
        return ActPolicy(1)


@dataclass(frozen=True)
class ActQuant:
    """backend.rs:786-806. kind: 0 Exact, 1 Bf16, 2 Fp8Row, 3 Nvfp4{divisor}."""

    kind: int = 0
    divisor: float = 0.0

    EXACT = 0
    BF16 = 1
    FP8_ROW = 2
    NVFP4 = 3

    def permitted(self, policy: ActPolicy) -> bool:
        """crates/velox-conformance/src/lib.rs:64-74."""
        if self.kind in (0, 1):
            return True
        if self.kind == 2:
            return policy.kind in (1, 2)
        return policy.kind == 2 and policy.divisor == self.divisor


@dataclass(frozen=True)
class WeightView:
    """Rows [row_begin, row_begin + rows) of an encoded parent [parent_rows, k] held in ``buf``
    (a uint8 device tensor with the parent's whole payload)."""

    buf: Any
    format: WeightFormat
    parent_rows: int
    k: int
    row_begin: int
    rows: int
    act: ActPolicy = ActPolicy()

    @staticmethod
    def full(buf, fmt: WeightFormat, n: int, k: int) -> "WeightView":
        return WeightView(buf, fmt, n, k, 0, n, ActPolicy())

    def with_act(self, act: ActPolicy) -> "WeightView":
        return replace(self, act=act)

    def rows_view(self, begin: int, rows: int) -> "WeightView":
        """``WeightView::rows`` (backend.rs:887-894)."""
        return replace(self, row_begin=self.row_begin + begin, rows=rows)


@dataclass(frozen=True)
class LinearPart:
    w: WeightView
    col: int


@dataclass
class LinearDst:
    y: Any
    ld: int
    parts: Sequence[LinearPart]


def swiglu_pair(gate: WeightView, up: WeightView):
    """backend.rs:2236-2270: the two views as one view of adjacent rows of one parent, with the
    gate and up column offsets of its output; None when they are not adjacent."""
    w = gate.rows
    same = (gate.buf is up.buf and gate.format == up.format and gate.parent_rows == up.parent_rows
            and gate.k == up.k and up.rows == w)
    act = gate.act.meet(up.act)
    if same and up.row_begin == gate.row_begin + w:
        return replace(gate, rows=2 * w, act=act), 0, w
    if same and gate.row_begin == up.row_begin + w:
        return replace(up, rows=2 * w, act=act), w, 0
    return None


def _need(what: str, have: int, want: int) -> None:
    if have < want:
        raise ShapeError(f"{what}: {have} elements, need {want}")


def check_weight(w: WeightView, buf_bytes: int) -> None:
    """check::weight (check.rs:100-116)."""
    w.format.check_shape(w.parent_rows, w.k)
    if w.rows <= 0 or w.row_begin < 0 or w.row_begin + w.rows > w.parent_rows:
        raise ShapeError(f"weight rows {w.row_begin}+{w.rows} outside parent of {w.parent_rows} rows")
    _need(f"{w.format.format_name} weight", (buf_bytes + 3) // 4,
          (w.format.payload_bytes(w.parent_rows, w.k) + 3) // 4)


def check_linear(x_len: int, w: WeightView, w_bytes: int, y_len: int, m: int) -> None:
    """check::linear (check.rs:118-131)."""
    if m <= 0:
        raise ShapeError("linear m must be non-zero")
    check_weight(w, w_bytes)
    _need("linear x", x_len, m * w.k)
    _need("linear y", y_len, m * w.rows)
