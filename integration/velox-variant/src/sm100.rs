//! `CudaKernels` for B200: the linear family on the sm_100a launchers of `kernels/velox_sm100.h`,
//! everything else on the portable kernels (the trait's defaults).
//!
//! Each override validates with `velox_core::check` exactly as the portable wrapper does
//! (crates/velox-cuda/src/portable.rs:236-260), makes one FFI call and maps the return code
//! with `velox_cuda::status` (crates/velox-cuda/src/lib.rs:95-112). A launcher that answers
//! `VELOX_ERR_UNSUPPORTED` (-1) for a format or shape it does not serve falls back to
//! `portable::*`, as the trait's contract asks (lib.rs:544-549).
//!
//! Not compiled: no Rust toolchain was available where this was written.

use std::ffi::c_void;

use velox_core::backend::{ActPolicy, ActQuant, LinearDst, NormKind, WeightView};
use velox_core::check::{self, to_i32};
use velox_core::{Error, Op, Result, WeightFormat};
use velox_cuda::portable::{self, format_code};
use velox_cuda::{status, CudaBuffer, CudaKernels};

const VELOX_ERR_UNSUPPORTED: i32 = -1;

// Policy and rounding codes of kernels/velox_sm100.h.
const POLICY_A16_ONLY: i32 = 0;
const POLICY_ALLOW_A8: i32 = 1;
const POLICY_ALLOW_A4: i32 = 2;
const ACT_EXACT: i32 = 0;
const ACT_BF16: i32 = 1;
const ACT_FP8_ROW: i32 = 2;
const ACT_NVFP4: i32 = 3;

/// `velox_sm100_view`.
#[repr(C)]
#[derive(Clone, Copy)]
struct View {
    w: *const u8,
    format: i32,
    policy: i32,
    n: i64,
    k: i64,
    row_begin: i64,
    rows: i32,
    divisor: f32,
}

/// `velox_sm100_part`.
#[repr(C)]
#[derive(Clone, Copy)]
struct Part {
    view: View,
    y: *mut f32,
    ld: i64,
    col: i64,
}

extern "C" {
    fn velox_sm100_linear_act(view: *const View, m: i32, divisor_out: *mut f32) -> i32;
    fn velox_sm100_linear_view(x: *const f32, view: *const View, m: i32, y: *mut f32, yb: *mut u16) -> i32;
    fn velox_sm100_linear_bf16(xb: *const u16, view: *const View, m: i32, y: *mut f32, yb: *mut u16) -> i32;
    fn velox_sm100_linear_swiglu(
        x: *const f32,
        gate: *const View,
        up: *const View,
        m: i32,
        out: *mut f32,
        outb: *mut u16,
    ) -> i32;
    fn velox_sm100_linear_swiglu_bf16(
        xb: *const u16,
        gate: *const View,
        up: *const View,
        m: i32,
        out: *mut f32,
        outb: *mut u16,
    ) -> i32;
    fn velox_sm100_linear_swiglu_act(gate: *const View, up: *const View, m: i32, divisor_out: *mut f32) -> i32;
    fn velox_sm100_linears(x: *const f32, xb: *const u16, parts: *const Part, nparts: i32, m: i32) -> i32;
    fn velox_sm100_matmul(x: *const f32, w: *const f32, y: *mut f32, m: i32, n: i32, k: i32) -> i32;
    fn velox_sm100_silu_mul(gate: *mut f32, up: *const f32, len: i64) -> i32;
    fn velox_sm100_add(acc: *mut f32, x: *const f32, len: i64) -> i32;
    fn velox_sm100_add_rms_norm_twin(
        acc: *mut f32,
        x: *const f32,
        weight: *const f32,
        y: *mut f32,
        yb: *mut u16,
        rows: i32,
        dim: i32,
        eps: f32,
        offset: i32,
    ) -> i32;
    fn velox_sm100_embed(
        ids: *const u32,
        count: i32,
        w: *const u8,
        format: i32,
        n: i64,
        k: i64,
        row_begin: i64,
        out: *mut f32,
    ) -> i32;
}

/// The formats the sm_100a launchers execute; everything else goes to the portable kernels.
fn served(f: WeightFormat) -> bool {
    match f {
        WeightFormat::Nvfp4 | WeightFormat::Fp8RowBf16 => true,
        WeightFormat::Ggml(t) => t == velox_core::ggml::GgmlType::Q4K,
        _ => false,
    }
}

fn view_of(w: &WeightView<'_, CudaBuffer>) -> Result<View> {
    let (policy, divisor) = match w.act {
        ActPolicy::A16Only => (POLICY_A16_ONLY, 0.0),
        ActPolicy::AllowA8 => (POLICY_ALLOW_A8, 0.0),
        ActPolicy::AllowA4 { divisor } => (POLICY_ALLOW_A4, divisor),
    };
    Ok(View {
        w: w.buf.as_ptr().cast(),
        format: format_code(w.format),
        policy,
        n: w.parent_rows as i64,
        k: w.k as i64,
        row_begin: w.row_begin as i64,
        rows: to_i32("rows", w.rows)?,
        divisor,
    })
}

fn act_of(code: i32, divisor: f32) -> Option<ActQuant> {
    match code {
        ACT_EXACT => Some(ActQuant::Exact),
        ACT_BF16 => Some(ActQuant::Bf16),
        ACT_FP8_ROW => Some(ActQuant::Fp8Row),
        ACT_NVFP4 => Some(ActQuant::Nvfp4 { divisor }),
        _ => None,
    }
}

/// bf16 twins live in f32 buffers, two values per slot (velox_core::backend, "bf16 twins").
fn twin_ptr(b: &CudaBuffer) -> *const u16 {
    b.as_ptr().cast()
}

fn twin_mut_ptr(b: &mut CudaBuffer) -> *mut u16 {
    b.as_mut_ptr().cast()
}

pub struct Sm100Kernels;

impl Sm100Kernels {
    fn act(&self, w: &WeightView<'_, CudaBuffer>, m: usize) -> Option<ActQuant> {
        if !served(w.format) {
            return None;
        }
        let v = view_of(w).ok()?;
        let m = i32::try_from(m).ok()?;
        let mut divisor = 0.0f32;
        // SAFETY: `v` and `divisor` are live locals; the call reads the view and launches nothing.
        let code = unsafe { velox_sm100_linear_act(&v, m, &mut divisor) };
        act_of(code, divisor)
    }
}

#[allow(clippy::too_many_arguments)]
impl CudaKernels for Sm100Kernels {
    fn native_ops(&self) -> &'static [Op] {
        &[Op::MatMul, Op::Linear, Op::LinearSwiglu, Op::SiluMul, Op::Add, Op::Embed]
    }

    fn matmul(&self, x: &CudaBuffer, w: &CudaBuffer, y: &mut CudaBuffer, m: usize, n: usize, k: usize) -> Result<()> {
        check::matmul(x.len(), w.len(), y.len(), m, n, k)?;
        let (mi, ni, ki) = (to_i32("m", m)?, to_i32("n", n)?, to_i32("k", k)?);
        // SAFETY: buffer extents validated above.
        match unsafe { velox_sm100_matmul(x.as_ptr(), w.as_ptr(), y.as_mut_ptr(), mi, ni, ki) } {
            VELOX_ERR_UNSUPPORTED => portable::matmul(x, w, y, m, n, k),
            code => status(code, "sm100 matmul"),
        }
    }

    fn linear(&self, x: &CudaBuffer, w: &WeightView<'_, CudaBuffer>, y: &mut CudaBuffer, m: usize) -> Result<()> {
        if !served(w.format) {
            return portable::linear(x, w, y, m);
        }
        check::linear(x.len(), w, w.buf.len(), y.len(), m)?;
        let v = view_of(w)?;
        // SAFETY: input, weight payload and output extents validated above.
        let code = unsafe { velox_sm100_linear_view(x.as_ptr(), &v, to_i32("m", m)?, y.as_mut_ptr(), std::ptr::null_mut()) };
        match code {
            VELOX_ERR_UNSUPPORTED => portable::linear(x, w, y, m),
            code => status(code, "sm100 linear"),
        }
    }

    fn linear_act(&self, w: &WeightView<'_, CudaBuffer>, m: usize) -> ActQuant {
        // (what `linear` above applies; the portable fallback is exact)
        self.act(w, m).unwrap_or(ActQuant::Exact)
    }

    fn serves_linears(&self, dsts: &[LinearDst<'_, '_, '_, CudaBuffer>], m: usize) -> bool {
        m > 0 && dsts.iter().all(|d| d.parts.iter().all(|p| served(p.w.format) && p.w.k % 64 == 0))
    }

    fn linears(
        &self,
        x: &CudaBuffer,
        xb: Option<&CudaBuffer>,
        _xq: Option<(&CudaBuffer, u32)>,
        dsts: &mut [LinearDst<'_, '_, '_, CudaBuffer>],
        m: usize,
    ) -> Result<()> {
        let mut parts = Vec::new();
        for d in dsts.iter_mut() {
            for p in d.parts {
                check::linear(x.len(), &p.w, p.w.buf.len(), d.y.len(), m)?;
                if p.col + p.w.rows > d.ld || d.y.len() < m * d.ld {
                    return Err(Error::Shape(format!(
                        "linears: columns {}..{} of {m} x {} in {} values",
                        p.col,
                        p.col + p.w.rows,
                        d.ld,
                        d.y.len()
                    )));
                }
                parts.push(Part { view: view_of(&p.w)?, y: d.y.as_mut_ptr(), ld: d.ld as i64, col: p.col as i64 });
            }
        }
        let xbp = xb.map_or(std::ptr::null(), twin_ptr);
        // SAFETY: every part's extents validated above; `parts` outlives the call, which copies
        // what it needs before returning.
        status(
            unsafe { velox_sm100_linears(x.as_ptr(), xbp, parts.as_ptr(), to_i32("parts", parts.len())?, to_i32("m", m)?) },
            "sm100 linears",
        )
    }

    fn takes_bf16(&self, w: &WeightView<'_, CudaBuffer>, m: usize) -> bool {
        self.act(w, m) == Some(ActQuant::Bf16)
    }

    fn linear_bf16(&self, xb: &CudaBuffer, w: &WeightView<'_, CudaBuffer>, y: &mut CudaBuffer, m: usize) -> Result<()> {
        // xb holds m * k bf16 values in (m * k + 1) / 2 slots
        check::linear(2 * xb.len(), w, w.buf.len(), y.len(), m)?;
        let v = view_of(w)?;
        // SAFETY: extents validated above.
        status(
            unsafe { velox_sm100_linear_bf16(twin_ptr(xb), &v, to_i32("m", m)?, y.as_mut_ptr(), std::ptr::null_mut()) },
            "sm100 linear_bf16",
        )
    }

    fn swiglu_twin(&self, gate: &WeightView<'_, CudaBuffer>, up: &WeightView<'_, CudaBuffer>, m: usize) -> bool {
        self.linear_swiglu_act(gate, up, m) == Some(ActQuant::Bf16)
    }

    fn linear_swiglu_twin(
        &self,
        xb: &CudaBuffer,
        gate: &WeightView<'_, CudaBuffer>,
        up: &WeightView<'_, CudaBuffer>,
        out: &mut CudaBuffer,
        outb: &mut CudaBuffer,
        m: usize,
    ) -> Result<()> {
        check::linear(2 * xb.len(), gate, gate.buf.len(), out.len(), m)?;
        check::linear(2 * xb.len(), up, up.buf.len(), out.len(), m)?;
        if 2 * outb.len() < m * gate.rows {
            return Err(Error::Shape(format!("linear_swiglu_twin outb: {} slots for {m} x {}", outb.len(), gate.rows)));
        }
        let (g, u) = (view_of(gate)?, view_of(up)?);
        // SAFETY: extents validated above.
        status(
            unsafe { velox_sm100_linear_swiglu_bf16(twin_ptr(xb), &g, &u, to_i32("m", m)?, out.as_mut_ptr(), twin_mut_ptr(outb)) },
            "sm100 linear_swiglu_twin",
        )
    }

    fn add_rms_norm_twin(
        &self,
        acc: &mut CudaBuffer,
        x: &CudaBuffer,
        weight: &CudaBuffer,
        y: &mut CudaBuffer,
        yb: &mut CudaBuffer,
        rows: usize,
        dim: usize,
        eps: f32,
        kind: NormKind,
    ) -> Result<()> {
        check::rms_norm(acc.len(), weight.len(), y.len(), rows, dim)?;
        check::rms_norm(x.len(), weight.len(), 2 * yb.len(), rows, dim)?;
        let offset = i32::from(kind == NormKind::Offset);
        // SAFETY: extents validated above.
        status(
            unsafe {
                velox_sm100_add_rms_norm_twin(
                    acc.as_mut_ptr(),
                    x.as_ptr(),
                    weight.as_ptr(),
                    y.as_mut_ptr(),
                    twin_mut_ptr(yb),
                    to_i32("rows", rows)?,
                    to_i32("dim", dim)?,
                    eps,
                    offset,
                )
            },
            "sm100 add_rms_norm_twin",
        )
    }

    fn linear_swiglu(
        &self,
        x: &CudaBuffer,
        gate: &WeightView<'_, CudaBuffer>,
        up: &WeightView<'_, CudaBuffer>,
        out: &mut CudaBuffer,
        m: usize,
    ) -> Result<()> {
        if !served(gate.format) || gate.format != up.format {
            return Err(Error::Unsupported("fused linear_swiglu".into()));   // the backend composes it
        }
        check::linear(x.len(), gate, gate.buf.len(), out.len(), m)?;
        check::linear(x.len(), up, up.buf.len(), out.len(), m)?;
        let (g, u) = (view_of(gate)?, view_of(up)?);
        // SAFETY: extents validated above.
        status(
            unsafe { velox_sm100_linear_swiglu(x.as_ptr(), &g, &u, to_i32("m", m)?, out.as_mut_ptr(), std::ptr::null_mut()) },
            "sm100 linear_swiglu",
        )
    }

    fn linear_swiglu_act(
        &self,
        gate: &WeightView<'_, CudaBuffer>,
        up: &WeightView<'_, CudaBuffer>,
        m: usize,
    ) -> Option<ActQuant> {
        if !served(gate.format) || gate.format != up.format || up.rows != gate.rows || up.k != gate.k {
            return None;
        }
        let (g, u) = (view_of(gate).ok()?, view_of(up).ok()?);
        let mut divisor = 0.0f32;
        // SAFETY: live locals; nothing is launched.
        let code = unsafe { velox_sm100_linear_swiglu_act(&g, &u, i32::try_from(m).ok()?, &mut divisor) };
        act_of(code, divisor)
    }

    fn embed(&self, ids: &[u32], table: &WeightView<'_, CudaBuffer>, out: &mut CudaBuffer) -> Result<()> {
        if !served(table.format) {
            return portable::embed(ids, table, out);
        }
        check::embed(ids, table, table.buf.len(), out.len())?;
        if ids.is_empty() {
            return Ok(());
        }
        // Host ids: staged to the device by the portable wrapper's path; the launcher here takes a
        // device pointer, so go through embed_from's buffer form when the ids are already there.
        portable::embed(ids, table, out)
    }

    fn embed_from(
        &self,
        ids: &CudaBuffer,
        offset: usize,
        count: usize,
        table: &WeightView<'_, CudaBuffer>,
        out: &mut CudaBuffer,
    ) -> Result<()> {
        if !served(table.format) || count == 0 {
            return portable::embed_from(ids, offset, count, table, out);
        }
        check::embed_from(ids.len(), offset, count, table, table.buf.len(), out.len())?;
        // SAFETY: extents validated above; ids are u32 values stored one per f32 slot.
        let code = unsafe {
            velox_sm100_embed(
                ids.as_ptr().cast::<u32>().add(offset),
                to_i32("count", count)?,
                table.buf.as_ptr().cast(),
                format_code(table.format),
                table.parent_rows as i64,
                table.k as i64,
                table.row_begin as i64,
                out.as_mut_ptr(),
            )
        };
        match code {
            VELOX_ERR_UNSUPPORTED => portable::embed_from(ids, offset, count, table, out),
            code => status(code, "sm100 embed"),
        }
    }

    fn silu_mul(&self, gate: &mut CudaBuffer, up: &CudaBuffer, len: usize) -> Result<()> {
        check::elementwise(gate.len(), up.len(), len)?;
        // SAFETY: extents validated above.
        status(unsafe { velox_sm100_silu_mul(gate.as_mut_ptr(), up.as_ptr(), len as i64) }, "sm100 silu_mul")
    }

    fn add(&self, acc: &mut CudaBuffer, x: &CudaBuffer, len: usize) -> Result<()> {
        check::elementwise(acc.len(), x.len(), len)?;
        // SAFETY: extents validated above.
        status(unsafe { velox_sm100_add(acc.as_mut_ptr(), x.as_ptr(), len as i64) }, "sm100 add")
    }
}

// Unused import guard for builds where no launcher takes an opaque pointer.
#[allow(dead_code)]
type Opaque = *mut c_void;
