"""A decoder's linear path as a tensor-parallel layer stack on NVFP4 weights.

Per layer, in the op order of the reference's ``Stack::forward`` (crates/velox-core/src/model.rs
:178-215) with attention replaced by a passthrough of the q projection::

    h = rms_norm(x)               q, k, v = linear(h)          (k, v computed, unused)
    x += all_reduce(linear(q, o)) h = rms_norm(x)
    g = silu(linear(h, gate)) * linear(h, up)                  (one fused launch)
    x += all_reduce(linear(g, down))

Tensor parallelism (absent from the reference, which is single-device): q/k/v/gate/up are split by
output rows (a rank keeps rows ``[r*N/p, (r+1)*N/p)`` re-based as a smaller parent with the same
per-tensor divisor); o/down are split along K (codes are a byte-aligned column slice, block
scales whole 512-byte atoms, same divisor: a re-layout of stored bytes, not a re-quantisation).
One all-reduce of the bf16 partial sums follows each row-split projection.

The geometry is the reference's ``qwen3-32b`` preset (crates/velox-core/src/plan.rs:59-72).
Weights are synthetic: N(0, 0.02^2) f32 per matrix from a per-(layer, projection) seed, quantised
on the device by ``encode_nvfp4``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .backend import Sm100Backend
from .weights import ActPolicy, ActQuant, WeightFormat, WeightView, align256

NV = WeightFormat.NVFP4


@dataclass(frozen=True)
class StackSpec:
    layers: int = 64
    hidden: int = 5120
    intermediate: int = 25600
    heads: int = 64
    kv_heads: int = 8
    head_dim: int = 128
    norm_eps: float = 1e-6

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def payload_bytes_per_layer(self) -> int:
        h, i, q, kv = self.hidden, self.intermediate, self.q_dim, self.kv_dim
        pb = NV.payload_bytes
        return pb(q, h) + 2 * pb(kv, h) + pb(h, q) + 2 * pb(i, h) + pb(h, i)

    def flops_per_token(self) -> int:
        h, i, q, kv = self.hidden, self.intermediate, self.q_dim, self.kv_dim
        return 2 * self.layers * (q * h + 2 * kv * h + h * q + 2 * i * h + h * i)


# Static activation divisors per use (the reference keeps one per projection in the artifact,
# `activation_input_divisor`): chosen so that e4m3(divisor * amax16 / 6) stays inside E4M3 for the
# activations each projection sees in this stack (unit-RMS norm output; q ~ N(0, 1.4^2);
# silu(g)*u with heavier tails).
DIV_NORM_OUT = 256.0
DIV_O_IN = 128.0
DIV_DOWN_IN = 16.0


def slice_rows_nvfp4(payload: torch.Tensor, n: int, k: int, begin: int, rows: int) -> torch.Tensor:
    """Rows [begin, begin+rows) of an NVFP4 parent as a parent of its own (column split).
    begin and rows are multiples of 128 so whole scale tiles move."""
    assert begin % 128 == 0 and rows % 128 == 0
    plane = align256(n * k // 2)
    out = torch.zeros(align256(NV.payload_bytes(rows, k)), dtype=torch.uint8, device=payload.device)
    out[: rows * k // 2] = payload[begin * k // 2:(begin + rows) * k // 2]
    oplane = align256(rows * k // 2)
    sb = begin * k // 16
    out[oplane:oplane + rows * k // 16] = payload[plane + sb:plane + sb + rows * k // 16]
    out[oplane + rows * k // 16:oplane + rows * k // 16 + 4] = payload[plane + n * k // 16:plane + n * k // 16 + 4]
    return out


def slice_k_nvfp4(payload: torch.Tensor, n: int, k: int, k_begin: int, k_len: int) -> torch.Tensor:
    """Columns [k_begin, k_begin+k_len) of an NVFP4 parent as a parent [n, k_len] (row split).
    k_begin and k_len are multiples of 64 so whole 512-byte scale atoms move."""
    assert k_begin % 64 == 0 and k_len % 64 == 0
    plane = align256(n * k // 2)
    out = torch.zeros(align256(NV.payload_bytes(n, k_len)), dtype=torch.uint8, device=payload.device)
    codes = payload[: n * k // 2].view(n, k // 2)[:, k_begin // 2:(k_begin + k_len) // 2]
    out[: n * k_len // 2] = codes.reshape(-1)
    atoms = payload[plane:plane + n * k // 16].view(n // 128, k // 64, 512)
    oplane = align256(n * k_len // 2)
    out[oplane:oplane + n * k_len // 16] = atoms[:, k_begin // 64:(k_begin + k_len) // 64, :].reshape(-1)
    out[oplane + n * k_len // 16:oplane + n * k_len // 16 + 4] = payload[plane + n * k // 16:plane + n * k // 16 + 4]
    return out


def fused_step_schedule(layers: int):
    """The launches of one fused tensor-parallel step in stream order, each with the flag row it
    waits on and the flag row it raises (-1: none): ``(op, layer, wait, signal)``.

    Rows per layer: 4l norm -> q|k|v ("blob rows written"), 4l+1 o -> norm ("partial sums landed"),
    4l+2 norm -> gate|up, 4l+3 down -> next norm; row 4*layers: finish -> end of step ("output rows
    written"). Every buffer another rank writes is protected in both directions by these waits: a
    norm overwrites the blob on all ranks only after each rank's row-split linear (which follows
    that rank's readers of the blob in its stream) has signalled, and a row-split linear
    overwrites the slots only after the norm that read them has signalled through the blob row."""
    P = TpFabric.PHASES_PER_LAYER
    ops = []
    for li in range(layers):
        p0 = P * li
        ops.append(("norm", li, p0 - 1 if li > 0 else -1, p0))
        ops.append(("qkv", li, p0, -1))
        ops.append(("o_scatter", li, -1, p0 + 1))
        ops.append(("norm", li, p0 + 1, p0 + 2))
        ops.append(("gate_up", li, p0 + 2, -1))
        ops.append(("down_scatter", li, -1, p0 + 3))
    last = P * layers
    ops.append(("finish", layers, last - 1, last))
    ops.append(("wait", layers, last, -1))
    return ops


class TpFabric:
    """Symmetric memory of a tensor-parallel group for the fused scatter / gather path: on every
    rank, one slot per source rank for bf16 partial sums of the rows this rank owns, the norm's
    NVFP4 blob for all rows, the final output, and a table of flags. Peers' copies are mapped into
    this process (torch symmetric memory: cuMem allocations exchanged once at set-up), so kernels
    store into them with ordinary addresses.

    Ordering between ranks, ``sync_mode``:
    ``"flags"``: every kernel that writes into other ranks' memory raises a flag there when it is
    done, every kernel that reads such data polls its own flags first;
    ``"kernel"``: the same flags raised and awaited by a one-warp barrier kernel between the
    phases (the data kernels carry no waits);
    ``"barrier"``: torch's signal-pad barrier kernels between the phases (kept for comparison; its
    device-side wait is not bounded).
    The first two use bounded waits that report through the status word (include/velox_sm100.h)."""

    PHASES_PER_LAYER = 4    # norm -> q|k|v, o -> norm, norm -> gate|up, down -> norm

    def __init__(self, backend: Sm100Backend, group, rank: int, world: int, m: int, hidden: int, layers: int,
                 sync_mode: str = "flags"):
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        assert m % (world * 128) == 0 and world <= 8
        assert sync_mode in ("flags", "kernel", "barrier")
        self.rank, self.world, self.m, self.hidden = rank, world, m, hidden
        self.sync_mode = sync_mode
        self.rows = m // world                               # token rows each rank owns
        self.phases = self.PHASES_PER_LAYER * layers + 1     # + "output rows written"
        slots_b, codes_b = world * self.rows * hidden * 2, m * hidden // 2
        atoms_b, out_b = m * hidden // 16, m * hidden * 2
        flags_b = self.phases * 8 * 4
        self.off_slots, self.off_codes = 0, align256(slots_b)
        self.off_atoms = self.off_codes + align256(codes_b)
        self.off_out = self.off_atoms + align256(atoms_b)
        self.off_flags = self.off_out + align256(out_b)
        total = self.off_flags + align256(flags_b)
        self.buf = symm.empty(total, dtype=torch.uint8, device=backend.device)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, group)
        # buffer_ptrs are the starts of the ranks' symmetric blocks; this tensor sits at the same
        # offset inside each of them
        inside = self.buf.data_ptr() - int(self.hdl.buffer_ptrs[rank])
        base = [int(p) + inside for p in self.hdl.buffer_ptrs]
        self.codes_ptrs = [p + self.off_codes for p in base]
        self.atoms_ptrs = [p + self.off_atoms for p in base]
        self.out_ptrs = [p + self.off_out for p in base]
        self.flag_ptrs = [p + self.off_flags for p in base]
        # this rank's slot in every owner's memory
        self.slot_ptrs = [p + self.off_slots + rank * self.rows * hidden * 2 for p in base]
        self.slots = self.buf[self.off_slots:self.off_slots + slots_b].view(torch.bfloat16)
        self.codes = self.buf[self.off_codes:self.off_codes + codes_b]
        self.atoms = self.buf[self.off_atoms:self.off_atoms + atoms_b]
        self.out = self.buf[self.off_out:self.off_out + out_b].view(torch.bfloat16)
        self.flags = self.buf[self.off_flags:self.off_flags + flags_b].view(torch.int32)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=backend.device)   # this rank's step counter
        self.maps = torch.zeros(world * 128, dtype=torch.uint8, device=backend.device)
        backend.tp_make_maps(self.maps, self.slot_ptrs, self.rows, hidden)
        self._lib = _lib
        self._syncs = {}
        torch.cuda.synchronize()
        self.hdl.barrier(channel=0)
        torch.cuda.synchronize()

    def sync(self, wait: int = -1, signal: int = -1):
        """The flags of one launch (row to wait on, row to raise; -1 none); None in barrier mode."""
        if self.sync_mode != "flags":
            return None
        key = (wait, signal)
        if key not in self._syncs:
            self._syncs[key] = self._make_sync(wait, signal)
        return self._syncs[key]

    def _make_sync(self, wait: int, signal: int):
        t = self._lib.TpSync()
        for i, p in enumerate(self.flag_ptrs):
            t.flag_tables[i] = p
        t.epoch = self.epoch.data_ptr()
        t.n, t.rank, t.wait_phase, t.signal_phase = self.world, self.rank, wait, signal
        return t

    def barrier(self, phase: int, backend: Sm100Backend) -> None:
        """The barrier between two phases in the modes that use one: this library's flag barrier on
        row ``phase``, or torch's signal-pad barrier."""
        if self.sync_mode == "kernel":
            key = ("barrier", phase)
            if key not in self._syncs:
                self._syncs[key] = self._make_sync(phase, phase)
            backend.tp_barrier(self._syncs[key])
        elif self.sync_mode == "barrier":
            self.hdl.barrier(channel=0)


@dataclass
class LayerWeights:
    q: WeightView
    k: WeightView
    v: WeightView
    o: WeightView
    gate: WeightView
    up: WeightView
    down: WeightView


class LinearStack:
    """The stack on one rank of a tensor-parallel group of ``world`` ranks."""

    def __init__(self, backend: Sm100Backend, spec: StackSpec, max_tokens: int, rank: int = 0,
                 world: int = 1, a4: bool = True, seed: int = 0, group=None, weights_of: "LinearStack" = None):
        self.b, self.spec, self.rank, self.world, self.group = backend, spec, rank, world, group
        self.max_tokens = max_tokens
        s = spec
        assert s.q_dim % (128 * world) == 0 and s.kv_dim % (128 * world) == 0
        assert s.intermediate % (128 * world) == 0
        dev = backend.device
        pol = (lambda d: ActPolicy.allow_a4(d)) if a4 else (lambda d: ActPolicy.a16_only())
        self.layers: List[LayerWeights] = []
        gen = torch.Generator(device=dev)
        if weights_of is not None:
            # a second set of activation buffers over the same weights (token chunks of one step)
            assert (weights_of.spec, weights_of.rank, weights_of.world, weights_of.a4) == (spec, rank, world, a4)
            self.layers = weights_of.layers
        for layer in range(s.layers if weights_of is None else 0):
            def make(proj: int, n: int, k: int) -> torch.Tensor:
                gen.manual_seed(seed * 1_000_003 + layer * 16 + proj)
                w = torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32) * 0.02
                return backend.encode_nvfp4(w)

            def col(proj, n, k, div):
                full = make(proj, n, k)
                rows = n // world
                buf = full if world == 1 else slice_rows_nvfp4(full, n, k, rank * rows, rows)
                return WeightView.full(buf, NV, rows, k).with_act(pol(div))

            def row(proj, n, k, div):
                full = make(proj, n, k)
                kl = k // world
                buf = full if world == 1 else slice_k_nvfp4(full, n, k, rank * kl, kl)
                return WeightView.full(buf, NV, n, kl).with_act(pol(div))

            self.layers.append(LayerWeights(
                q=col(0, s.q_dim, s.hidden, DIV_NORM_OUT), k=col(1, s.kv_dim, s.hidden, DIV_NORM_OUT),
                v=col(2, s.kv_dim, s.hidden, DIV_NORM_OUT), o=row(3, s.hidden, s.q_dim, DIV_O_IN),
                gate=col(4, s.intermediate, s.hidden, DIV_NORM_OUT),
                up=col(5, s.intermediate, s.hidden, DIV_NORM_OUT),
                down=row(6, s.hidden, s.intermediate, DIV_DOWN_IN)))
        m = max_tokens
        bf, f32 = torch.bfloat16, torch.float32
        self.norm_w = torch.ones(s.hidden, dtype=f32, device=dev)
        self.x = torch.zeros(m * s.hidden, dtype=f32, device=dev)       # residual stream
        self.hb = torch.zeros(m * s.hidden, dtype=bf, device=dev)       # norm output (bf16 twin)
        self.qb = torch.zeros(m * s.q_dim // world, dtype=bf, device=dev)
        self.kb = torch.zeros(m * s.kv_dim // world, dtype=bf, device=dev)
        self.vb = torch.zeros(m * s.kv_dim // world, dtype=bf, device=dev)
        self.gb = torch.zeros(m * s.intermediate // world, dtype=bf, device=dev)
        self.pb = torch.zeros(m * s.hidden, dtype=bf, device=dev)       # row-split partial sums
        self.outb = torch.zeros(m * s.hidden, dtype=bf, device=dev)
        self.a4 = a4
        self.hq = backend.q4_blob(m, s.hidden)                          # norm output as NVFP4
        self.qq = backend.q4_blob(m, s.q_dim // world)                  # q projection as NVFP4 (o's input)
        self.gq = backend.q4_blob(m, s.intermediate // world)           # silu(gate)*up as NVFP4 (down's input)
        self.fabric: Optional[TpFabric] = None
        self.weight_bytes = sum(v.buf.numel() for l in self.layers
                                for v in (l.q, l.k, l.v, l.o, l.gate, l.up, l.down))

    def _all_reduce(self, t: torch.Tensor) -> None:
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)

    # -- q, k, v of one input: one launch at every width (the streaming kernel at decode sizes, one
    #    persistent GEMM grid over the tiles of all three views at prefill sizes).
    def _qkv(self, l: LayerWeights, hq, m: int, emit: bool, sync=None) -> None:
        b = self.b
        qpart = (l.q, None, self.qq, DIV_O_IN) if emit else (l.q, self.qb, None, 0.0)
        parts = [qpart, (l.k, self.kb, None, 0.0), (l.v, self.vb, None, 0.0)]
        if sync is not None:
            b.tp_linears_q4(hq, DIV_NORM_OUT, parts, m, sync)
        else:
            b.linears_q4(hq, DIV_NORM_OUT, parts, m)

    def enable_fused_tp(self, m: int, sync_mode: str = "flags") -> bool:
        """Set up the symmetric buffers of the fused scatter / gather path for steps of m tokens.
        False (and nothing changed) where it does not apply."""
        if self.world == 1 or not self.a4 or m <= 16 or m % (self.world * 128) != 0 or m > self.max_tokens:
            return False
        self.fabric = TpFabric(self.b, self.group if self.group is not None else torch.distributed.group.WORLD,
                               self.rank, self.world, m, self.spec.hidden, self.spec.layers, sync_mode)
        return True

    def forward_fused_tp(self, xb_in: torch.Tensor, own_rows_only: bool = False) -> torch.Tensor:
        """The step with communication fused into the kernels on either side of it. Token rows
        are owned by ranks in equal blocks. o and down store their bf16 partial tiles straight into
        the owning rank's slots (GEMM epilogue, TMA stores over NVLink) and raise a flag there; the
        norm waits for the flags, adds the slots to its own rows of the f32 residual, normalises
        them, writes the NVFP4 result into every rank's blob and raises the flag the next linears
        wait for. ``xb_in`` is [m, hidden] bf16, or with ``own_rows_only`` just this rank's
        [m / world, hidden] rows of it (all the step reads)."""
        b, s, f = self.b, self.spec, self.fabric
        h, m, rows, world = s.hidden, f.m, f.rows, self.world
        r0 = self.rank * rows
        launches0 = b.launch_count()
        x_own = self.x[: rows * h]
        src = xb_in.reshape(-1)
        x_own.copy_(src[: rows * h] if own_rows_only else src[r0 * h:(r0 + rows) * h])
        hq = (f.codes, f.atoms)
        flags = f.sync_mode == "flags"
        if f.sync_mode != "barrier":
            b.tp_step_begin(f.epoch)
        nslots = 0
        for op, li, wait, signal in fused_step_schedule(len(self.layers)):
            sync = f.sync(wait, signal)                   # None unless the kernels carry the flags themselves
            l = self.layers[li] if li < len(self.layers) else None
            if op == "norm":
                b.tp_norm_q4(x_own, f.slots, nslots, rows * h, self.norm_w, f.codes_ptrs, f.atoms_ptrs, r0, rows, h,
                             s.norm_eps, DIV_NORM_OUT, sync=sync)
                nslots = world
                f.barrier(signal, b)                      # every rank's rows of the blob are in place
            elif op == "qkv":
                self._qkv(l, hq, m, True, sync=sync)
            elif op == "gate_up":
                if flags:
                    b.tp_linear_swiglu_q4_to_q4(hq, DIV_NORM_OUT, l.gate, l.up, m, self.gq, DIV_DOWN_IN, sync=sync)
                else:
                    b.linear_swiglu_q4_to_q4(hq, DIV_NORM_OUT, l.gate, l.up, m, self.gq, DIV_DOWN_IN)
            elif op == "o_scatter":
                b.tp_linear_q4_scatter(self.qq, DIV_O_IN, l.o, m, f.maps, rows, sync=sync)
                f.barrier(signal, b)                      # all partial sums of o have landed
            elif op == "down_scatter":
                b.tp_linear_q4_scatter(self.gq, DIV_DOWN_IN, l.down, m, f.maps, rows, sync=sync)
                f.barrier(signal, b)
            elif op == "finish":
                b.tp_finish(x_own, f.slots, world, rows * h, f.out_ptrs, r0, rows, h, sync=sync)
                f.barrier(signal, b)
            elif op == "wait" and flags:
                b.tp_wait(sync)                           # every rank's rows of the output are in place
        self.launches_per_step = b.launch_count() - launches0
        return f.out

    def forward_gathered(self, xb_in: torch.Tensor, m: int) -> torch.Tensor:
        """The sharded step with library collectives only and the fused step's arithmetic: after
        each row-split projection the ranks' bf16 partial sums are all-gathered and added in rank
        order in f32 (what the fused norm does with its slots) to a replicated residual, so every
        value equals ``forward_fused_tp``'s bit for bit. The checker of the fused step, and the step
        to use where symmetric memory is not available."""
        b, s = self.b, self.spec
        h, world = s.hidden, self.world
        assert self.a4 and 16 < m <= self.max_tokens
        self.x[: m * h].copy_(xb_in.reshape(-1)[: m * h])
        if not hasattr(self, "_gather"):
            self._gather = torch.zeros(world, self.max_tokens * h, dtype=torch.bfloat16, device=b.device)
            self._part = torch.zeros(self.max_tokens * h, dtype=torch.float32, device=b.device)

        def summed():
            """sum over ranks, in rank order, of the bf16 partial sums in pb"""
            if world > 1:
                torch.distributed.all_gather_into_tensor(self._gather.view(-1), self.pb, group=self.group)
            else:
                self._gather[0].copy_(self.pb)
            part = self._part
            part.copy_(self._gather[0])
            for r in range(1, world):
                part += self._gather[r]
            return part

        part = None
        for l in self.layers:
            b.add_rms_norm_q4(self.x, part, self.norm_w, None, self.hq, m, h, s.norm_eps, DIV_NORM_OUT)
            self._qkv(l, self.hq, m, True)
            b.linear_q4(self.qq, DIV_O_IN, l.o, None, m, yb=self.pb)
            part = summed()
            b.add_rms_norm_q4(self.x, part, self.norm_w, None, self.hq, m, h, s.norm_eps, DIV_NORM_OUT)
            b.linear_swiglu_q4_to_q4(self.hq, DIV_NORM_OUT, l.gate, l.up, m, self.gq, DIV_DOWN_IN)
            b.linear_q4(self.gq, DIV_DOWN_IN, l.down, None, m, yb=self.pb)
            part = summed()
        b.add(self.x, part, m * h)
        return b.bf16_twin_into(self.x, self.outb, m * h)

    def forward(self, xb_in: torch.Tensor, m: int) -> torch.Tensor:
        """One step over m tokens: xb_in is bf16 [m, hidden] on the device; returns the final
        residual stream rounded to bf16 ([m, hidden], device)."""
        b, s = self.b, self.spec
        h = s.hidden
        assert m <= self.max_tokens
        launches0 = b.launch_count()
        self.x[: m * h].copy_(xb_in.reshape(-1)[: m * h])
        first = True
        # the norm hands the FP4 linears their quantised input directly, and the linears that feed
        # another linear emit its FP4 input from their epilogue
        q4 = self.a4 and b.linear_act(self.layers[0].q, m).kind == ActQuant.NVFP4
        emit = q4
        for l in self.layers:
            # x (+= previous down partial), h = rms_norm(x)
            if q4:
                b.add_rms_norm_q4(self.x, None, self.norm_w, None, self.hq, m, h, s.norm_eps, DIV_NORM_OUT,
                                  xb=None if first else self.pb)
                # q feeds o directly (attention passthrough), so it is produced as o's FP4 input
                self._qkv(l, self.hq, m, emit)
            else:
                b.add_rms_norm_twin(self.x, None, self.norm_w, None, self.hb, m, h, s.norm_eps,
                                    xb=None if first else self.pb)
                b.linear_bf16(self.hb, l.q, None, m, yb=self.qb)
                b.linear_bf16(self.hb, l.k, None, m, yb=self.kb)
                b.linear_bf16(self.hb, l.v, None, m, yb=self.vb)
            first = False
            if emit:
                b.linear_q4(self.qq, DIV_O_IN, l.o, None, m, yb=self.pb)
            else:
                b.linear_bf16(self.qb, l.o, None, m, yb=self.pb)   # attention passthrough: a = q
            self._all_reduce(self.pb[: m * h])
            if q4:
                b.add_rms_norm_q4(self.x, None, self.norm_w, None, self.hq, m, h, s.norm_eps, DIV_NORM_OUT,
                                  xb=self.pb)
                if emit:
                    b.linear_swiglu_q4_to_q4(self.hq, DIV_NORM_OUT, l.gate, l.up, m, self.gq, DIV_DOWN_IN)
                    b.linear_q4(self.gq, DIV_DOWN_IN, l.down, None, m, yb=self.pb)
                else:
                    b.linear_swiglu_q4(self.hq, DIV_NORM_OUT, l.gate, l.up, None, self.gb, m)
                    b.linear_bf16(self.gb, l.down, None, m, yb=self.pb)
            else:
                b.add_rms_norm_twin(self.x, None, self.norm_w, None, self.hb, m, h, s.norm_eps, xb=self.pb)
                b.linear_swiglu_twin(self.hb, l.gate, l.up, None, self.gb, m)
                b.linear_bf16(self.gb, l.down, None, m, yb=self.pb)
            self._all_reduce(self.pb[: m * h])
        b.add_bf16(self.x, self.pb, m * h)
        out = b.bf16_twin_into(self.x, self.outb, m * h)
        self.launches_per_step = b.launch_count() - launches0   # this library's kernels per step
        return out


class ChunkedStack:
    """The fused tensor-parallel step over token chunks that run side by side: the step's tokens are
    cut into ``chunks`` equal parts, each with its own activation buffers, symmetric memory and
    stream, all over one set of weights. A token's result does not depend on which other tokens
    share its launch, so the outputs are those of the unchunked step bit for bit; what changes is
    the schedule: while one chunk's row-split linear waits for its partial sums to cross the links
    (its CTAs have exited, its stores are in flight), another chunk's kernels have the SMs. Worth it
    where the links' time is comparable with the compute (many ranks), at the price of reading the
    weights once per chunk."""

    def __init__(self, backend: Sm100Backend, spec: StackSpec, max_tokens: int, rank: int, world: int,
                 chunks: int = 2, seed: int = 0, group=None):
        assert chunks >= 1 and max_tokens % (chunks * world * 128) == 0
        self.b, self.spec, self.rank, self.world, self.chunks = backend, spec, rank, world, chunks
        self.m = max_tokens
        mc = max_tokens // chunks
        first = LinearStack(backend, spec, mc, rank, world, True, seed, group)
        self.parts = [first] + [LinearStack(backend, spec, mc, rank, world, True, seed, group, weights_of=first)
                                for _ in range(chunks - 1)]
        self.streams = [torch.cuda.Stream(device=backend.device) for _ in range(chunks)]
        self.weight_bytes = first.weight_bytes
        self.layers = first.layers
        self.out = torch.zeros(max_tokens * spec.hidden, dtype=torch.bfloat16, device=backend.device)
        self.launches_per_step = 0

    def enable_fused_tp(self, m: int, sync_mode: str = "kernel") -> bool:
        assert m == self.m
        if sync_mode == "flags":
            # Kernels that hold every SM while they wait for a peer must not share a GPU with the
            # other chunk's kernels the peer is waiting for in turn; barriers between the phases
            # are one-warp kernels and cannot starve anything.
            raise ValueError("chunks run with barrier kernels between the phases ('kernel' or 'barrier')")
        return all(p.enable_fused_tp(m // self.chunks, sync_mode) for p in self.parts)

    def forward_fused_tp(self, xb_in: torch.Tensor) -> torch.Tensor:
        """xb_in: [m, hidden] bf16 on the device; returns the whole output [m, hidden] (every rank)."""
        h, mc = self.spec.hidden, self.m // self.chunks
        main = torch.cuda.current_stream(self.b.device)
        start = torch.cuda.Event()
        start.record(main)
        launches = 0
        for c, (p, st) in enumerate(zip(self.parts, self.streams)):
            st.wait_event(start)
            with torch.cuda.stream(st):
                out = p.forward_fused_tp(xb_in.reshape(-1)[c * mc * h:(c + 1) * mc * h])
                self.out[c * mc * h:(c + 1) * mc * h].copy_(out.view(-1)[: mc * h])
                done = torch.cuda.Event()
                done.record(st)
            main.wait_event(done)
            launches += p.launches_per_step
        self.launches_per_step = launches
        return self.out
