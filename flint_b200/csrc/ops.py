"""Python face of the CUDA kernels: one method per kernel, taking torch tensors.

``CudaOps`` checks types and shapes, hands raw pointers and the current stream to the
``extern "C"`` launchers and raises ``KernelError`` with the launcher's message on any
refusal.  It has no fallback: on a machine without the compiled extension or without
a CUDA device it raises.  The reference wraps its shaders the same way, one function
per shader building the scalar and binding lists (crates/thuban_model/src/ops/*.rs).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from ..errors import KernelError
from . import build

F32, BF16 = 0, 1


def _raw_stream(device_index) -> int:
    """Handle of the device's current stream."""
    fast = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if fast is not None:
        return fast(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


def _code(dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(t, name, dtype=None, dims=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dims, got shape {tuple(t.shape)}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


@dataclass
class MoePlan:
    """Rows sorted by expert: where each (token, choice) went and which expert owns each
    row tile.  All tensors live on the device; nothing is read back."""
    n_experts: int
    tile_rows: int
    max_tiles: int
    counts: torch.Tensor       # [E]
    offsets: torch.Tensor      # [E+1]
    row_of: torch.Tensor       # [T, top] sorted row of (token, choice)
    token_of: torch.Tensor     # [top T] token of each sorted row
    tile_expert: torch.Tensor  # [max_tiles]
    tile_row0: torch.Tensor    # [max_tiles]
    n_tiles: torch.Tensor      # [1]
    top: int = 2               # choices per token


class CudaOps:
    """The kernel set on one CUDA device."""

    name = "cuda"

    def __init__(self, device="cuda:0"):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: flint_b200 runs on the GPU only and has no CPU fallback")
        self.device = torch.device(device)
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        # launch plans are sized for the device: so many blocks or warps per multiprocessor
        self.sm_count = int(torch.cuda.get_device_properties(self.device).multi_processor_count)
        self._libs = {}
        self.launches = 0
        self._profile = None
        self._label = None          # what the next launch works on (profiles list products by their shape)
        # One buffer for what the host reads back after a step, so that one copy brings all of it: a flag set by
        # a tensor-core kernel whose bounded wait ran out, a flag set by a kernel that met a position without a
        # page, and the sampled tokens.
        self.MAX_TOKEN_ROWS = 4096
        self.readback = torch.zeros(2 + self.MAX_TOKEN_ROWS, dtype=torch.int32, device=self.device)
        self.tc_error = self.readback[0:1]
        self.page_error = self.readback[1:2]
        self.token_out = self.readback[2:]
        # arrival counters of the decode attention kernels (one per row, kv head and chunk of query heads): zero
        # between launches; a launch that gave up a wait may leave some set, so they are cleared with its flag
        self.attention_arrivals = torch.zeros(1 << 15, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ plumbing
    def _fn(self, module, name):
        lib = self._libs.get(module)
        if lib is None:
            lib = build.load_module(module)
            getattr(lib, f"flint_{module}_last_error").restype = ctypes.c_char_p
            self._libs[module] = lib
        return getattr(lib, name)

    def _stream(self):
        """The current stream of the device as the launchers take it.  Asked for at every launch (a graph is
        captured on a stream of its own), through the call that returns the bare handle: building a stream
        object each time cost 7 us of the 25 us a launch takes on the host."""
        return c_void_p(_raw_stream(self._device_index))

    def _run(self, module, name, *args):
        fn = self._fn(module, name)
        if self._profile is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args, self._stream())
            e1.record()
            self._profile.append((name + (" " + self._label if self._label else ""), e0, e1))
        else:
            rc = fn(*args, self._stream())
        self._label = None
        self.launches += 1
        if rc != 0:
            msg = getattr(self._libs[module], f"flint_{module}_last_error")()
            raise KernelError((msg or b"unknown kernel error").decode())

    # Per-kernel device times, like the reference's timestamp profiler
    # (crates/thuban_profiler/src/lib.rs:173-248): events around every launch, summed by name.
    def start_profile(self):
        self._profile = []

    def stop_profile(self, ordered=False):
        """Returns {kernel name: (launches, total ms)} and stops profiling; ``ordered``: the launches in order
        instead, [(kernel name, ms)]."""
        torch.cuda.synchronize(self.device)
        if ordered:
            out = [(name, e0.elapsed_time(e1)) for name, e0, e1 in self._profile or []]
            self._profile = None
            return out
        out = {}
        for name, e0, e1 in self._profile or []:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1))
        self._profile = None
        return out

    def wait_probe(self, limit_cycles=1_000_000):
        """Launch a kernel whose one wait, on a barrier nobody arrives at, runs out after ``limit_cycles`` clock
        cycles: it raises the same flag as a product kernel whose wait ran out, and returns.  Nothing faults or
        hangs.  For tests of the path from a kernel that gave up to the host's error."""
        self._run("gemm_tc", "flint_gemm_tc_wait_probe", c_longlong(int(limit_cycles)), _ptr(self.tc_error))

    def set_wait_cycles(self, cycles=0):
        """The limit (clock cycles) of every bounded wait in later launches of the tensor-core kernels;
        0 restores the default of about two seconds."""
        for module in ("gemm_tc", "attention_tc"):
            fn = self._fn(module, f"flint_{module}_set_wait_cycles")
            fn.restype = None
            fn(c_longlong(int(cycles)))

    def preload(self, modules=None):
        """Compile and load modules ahead of their first use."""
        mods = list(modules or build.available_modules())
        build.compile_all(mods)
        for m in mods:
            if m in build.MODULES:              # the host runtime is loaded by its own face
                self._fn(m, f"flint_{m}_last_error")

    # ------------------------------------------------------------------ row-wise
    def embed(self, ids, table, out, scale=1.0, fed_rows=None, fed_from=None):
        """Rows of the table by token id.  ``fed_rows`` [T] with ``fed_from``: where a row's entry is not
        negative, its token is read from that place of ``fed_from`` (tokens sampled on the device that the
        host has not read yet) instead of ``ids``."""
        _check(ids, "ids", torch.int32, 1)
        _check(table, "table", dims=2)
        _check(out, "out", torch.float32, 2)
        T, (V, H) = ids.numel(), table.shape
        if tuple(out.shape) != (T, H):
            raise KernelError(f"embed: out must be [{T}, {H}]")
        if (fed_rows is None) != (fed_from is None):
            raise KernelError("embed: fed rows and their source come together")
        if fed_rows is not None:
            _check(fed_rows, "fed_rows", torch.int32, 1)
            _check(fed_from, "fed_from", torch.int32, 1)
            if fed_rows.numel() != T:
                raise KernelError(f"embed: fed_rows must have {T} entries")
        self._run("elementwise", "flint_embed", _ptr(ids), _ptr(fed_rows), _ptr(fed_from), _ptr(table),
                  c_int(_code(table.dtype)), _ptr(out), c_int(T), c_int(H), c_int(V), c_float(scale))

    def norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None):
        """mode 'layer' or 'rms'; writes float32 and/or bfloat16 copies of the result."""
        _check(x, "x", torch.float32, 2)
        H = x.shape[1]
        rows = row_index.numel() if row_index is not None else x.shape[0]
        _check(gamma, "gamma", torch.float32, 1)
        if gamma.numel() != H or (beta is not None and (beta.numel() != H or beta.dtype != torch.float32)):
            raise KernelError("norm: scale and bias must be float32 of the row width")
        for o, dt in ((out_f32, torch.float32), (out_bf16, torch.bfloat16)):
            if o is not None:
                _check(o, "norm output", dt, 2)
                if tuple(o.shape) != (rows, H):
                    raise KernelError(f"norm: output must be [{rows}, {H}]")
        if row_index is not None:
            _check(row_index, "row_index", torch.int32, 1)
        self._run("elementwise", "flint_norm", _ptr(x), _ptr(row_index), _ptr(gamma), _ptr(beta), c_float(eps),
                  c_int({"layer": 0, "rms": 1}[mode]), _ptr(out_f32), _ptr(out_bf16), c_int(rows), c_int(H))

    def row_norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None, pending=None,
                 router=None):
        """Norm of the residual rows with what is pending applied first (x is updated in place) and,
        on request, the routing of every row.  Falls back to separate kernels for widths that the
        fused kernel does not take."""
        _check(x, "x", torch.float32, 2)
        T, H = x.shape
        if H % 4 or H > 16384 or (router is not None and (row_index is not None or H * 4 > 160000
                                                          or router.weight.shape[0] > H
                                                          or (getattr(router, "rule", "") == "sigmoid_grouped"
                                                              and 2 * router.weight.shape[0] > H))):
            if pending is not None:
                self.apply_pending(x, pending)
            tmp = out_f32
            if router is not None and tmp is None:
                tmp = torch.empty((T, H), dtype=torch.float32, device=x.device)
            self.norm(x, gamma, beta, eps, mode, out_f32=tmp, out_bf16=out_bf16, row_index=row_index)
            if router is not None:
                self.route(tmp, router)
            return
        rows = row_index.numel() if row_index is not None else T
        for o, dt in ((out_f32, torch.float32), (out_bf16, torch.bfloat16)):
            if o is not None:
                _check(o, "norm output", dt, 2)
                if tuple(o.shape) != (rows, H):
                    raise KernelError(f"row_norm: output must be [{rows}, {H}]")
        if gamma is not None and (gamma.dtype != torch.float32 or gamma.numel() != H):
            raise KernelError("row_norm: scale must be float32 of the row width")
        partials = bias = y = row_of = gts = None
        S, stride, top = 0, 0, 0
        if pending is not None:
            if pending.partials is not None:
                partials = pending.partials
                _check(partials, "pending partials", torch.float32, 3)
                if tuple(partials.shape[1:]) != (T, H):
                    raise KernelError("row_norm: pending partial sums do not match the residual")
                S, stride, bias = partials.shape[0], partials.stride(0), pending.bias
            if pending.y is not None:
                y, row_of, gts = pending.y, pending.row_of, pending.gates
                _check(y, "pending expert rows", torch.float32, 2)
                top = row_of.numel() // max(T, 1)
                if y.shape[1] != H or top < 1 or row_of.numel() != top * T or gts.numel() != top * T:
                    raise KernelError("row_norm: pending expert rows do not match the residual")
        wr = logits = None
        E, jit, ids, gates = 0, 0.0, None, None
        r_top, r_groups, r_keep, r_scale = 0, 1, 1, 1.0
        r_rule, r_extra, r_aux = 0, 0, None
        r_corr, r_norm = None, 0
        if router is not None:
            wr, E, jit, ids, gates = router.weight, router.weight.shape[0], router.jitter_eps, router.expert_ids, router.gates
            logits = getattr(router, "logits", None)
            r_top, r_groups = int(getattr(router, "top", 0)), int(getattr(router, "groups", 1))
            r_keep, r_scale = int(getattr(router, "keep", 1)), float(getattr(router, "scale", 1.0))
            if logits is not None:
                _check(logits, "router logits", torch.float32, 2)
                if tuple(logits.shape) != (T, E):
                    raise KernelError(f"row_norm: router logits must be [{T}, {E}]")
            _check(wr, "router weight", dims=2)
            if wr.shape[1] != H or ids.numel() != (r_top or 2) * T or gates.numel() != (r_top or 2) * T:
                raise KernelError("row_norm: router shapes do not match")
            if getattr(router, "rule", "") == "sigmoid":
                r_rule, r_extra, r_aux = 1, int(router.extra), router.weights
                _check(r_aux, "router weights out", torch.float32, 2)
                if tuple(r_aux.shape) != (T, r_top + r_extra) or r_top < 1:
                    raise KernelError(f"row_norm: the sigmoid router's weights must be [{T}, {r_top + r_extra}]")
            elif getattr(router, "rule", "") == "sigmoid_grouped":
                r_rule, r_corr, r_norm = 2, router.correction, 1 if router.normalize else 0
                if r_corr is not None and (r_corr.dtype != torch.float32 or r_corr.numel() != E):
                    raise KernelError("row_norm: the router's correction must be float32, one per expert")
        self._run("row_fused", "flint_row_norm", _ptr(x), _ptr(row_index), c_int(rows), c_int(H), _ptr(partials),
                  c_int(S), c_longlong(stride), _ptr(bias), _ptr(y), _ptr(row_of), _ptr(gts), c_int(top), _ptr(gamma), _ptr(beta),
                  c_float(eps), c_int({"layer": 0, "rms": 1}[mode]), _ptr(out_f32), _ptr(out_bf16), _ptr(wr),
                  c_int(_code(wr.dtype) if wr is not None else 0), c_int(E), c_float(jit), _ptr(ids), _ptr(gates),
                  _ptr(logits), c_int(r_top), c_int(r_groups), c_int(r_keep), c_float(r_scale), c_int(r_rule), c_int(r_extra),
                  _ptr(r_aux), _ptr(r_corr), c_int(r_norm))

    def apply_pending(self, x, pending):
        """x += what a part left pending (for a norm that cannot take it along)."""
        _check(x, "x", torch.float32, 2)
        T, H = x.shape
        if H % 4 == 0 and H <= 16384:
            return self.row_norm(x, None, None, 0.0, "layer", pending=pending)
        if pending.partials is not None:
            p = pending.partials
            self._run("elementwise", "flint_add_partials", _ptr(x), _ptr(p), c_int(p.shape[0]), c_longlong(p.stride(0)),
                      _ptr(pending.bias), c_int(T), c_int(H))
        if pending.y is not None:
            self.moe_combine(x, pending.y, pending.row_of, pending.gates)

    def rope_kv_write(self, qkv, pos, slot, cos, sin, rot, q_out, cache, nq, nkv, hd, write_kv, status, bias=None,
                      style="half"):
        """qkv [T, W] or [S, T, W] float32 (S partial sums that are added here, with the bias).  ``style``: which
        dims of a head rotate together: "half" (i and i + rot/2) or "interleaved" (2i and 2i + 1)."""
        if style not in ("half", "interleaved"):
            raise KernelError(f"rope_kv_write: unknown rotation style {style!r}")
        if qkv.dim() == 2:
            qkv = qkv.unsqueeze(0)
        _check(qkv, "qkv", torch.float32, 3)
        S, T = qkv.shape[0], qkv.shape[1]
        if qkv.shape[2] != (nq + 2 * nkv) * hd:
            raise KernelError("rope_kv_write: qkv width does not match the head counts")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != qkv.shape[2]):
            raise KernelError("rope_kv_write: bias must be float32 of the qkv width")
        _check(q_out, "q_out", dims=2)
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if cos.shape[1] * 2 != rot and rot > 0:
            raise KernelError("rope_kv_write: table width must be rot/2")
        if cache is not None:
            k, v, bt, P = cache.k, cache.v, cache.block_table, cache.page_size
            cdt = _code(k.dtype)
            if tuple(k.shape[1:]) != (nkv, P, hd) or tuple(v.shape[1:]) != (nkv, P, hd):
                raise KernelError(f"rope_kv_write: cache pages are {tuple(k.shape[1:])} and {tuple(v.shape[1:])}, "
                                  f"expected {(nkv, P, hd)} for both")
            max_pages = bt.shape[1]
        else:
            if write_kv:
                raise KernelError("rope_kv_write: no cache to write to")
            k = v = bt = None
            cdt, P, max_pages = F32, 16, 0
        self._run("elementwise", "flint_rope_kv_write", _ptr(qkv), _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin),
                  c_int(rot), c_int(1 if style == "interleaved" else 0), _ptr(q_out), c_int(_code(q_out.dtype)), _ptr(k),
                  _ptr(v), c_int(cdt), _ptr(bt),
                  c_int(max_pages), c_int(P), c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(1 if write_kv else 0),
                  _ptr(status), c_int(S), c_longlong(qkv.stride(0)), _ptr(bias))

    def gather_rows(self, x, index, out):
        _check(x, "x", dims=2)
        _check(index, "index", torch.int32, 1)
        _check(out, "out", x.dtype, 2)
        if out.shape[0] != index.numel() or out.shape[1] != x.shape[1]:
            raise KernelError("gather_rows: output shape does not match")
        self._run("elementwise", "flint_gather_rows", _ptr(x), _ptr(index), _ptr(out), c_int(index.numel()),
                  c_int(x.shape[1] * x.element_size()))

    def moe_combine(self, h, y, row_of, gates):
        _check(h, "h", torch.float32, 2)
        _check(y, "y", torch.float32, 2)
        T, H = h.shape
        top = row_of.numel() // max(T, 1)
        if y.shape[1] != H or top < 1 or row_of.numel() != top * T or gates.numel() != top * T:
            raise KernelError("moe_combine: shapes do not match")
        self._run("elementwise", "flint_moe_combine", _ptr(h), _ptr(y), _ptr(row_of), _ptr(gates), c_int(T), c_int(H),
                  c_int(top))

    # ------------------------------------------------------------------ matrix products
    def gemm(self, x, w, out, bias=None, accumulate=False):
        """out = x @ w.T (+ bias) (+ out).  x [M,K], w [N,K], out [M,N]."""
        self._gemm(x, w, False, out, bias, accumulate, "silu", None)

    GATE_BLOCK = 16     # rows per block of the paired gate/up layout (GATE_BLOCK in common.cuh)

    @classmethod
    def paired_rows(cls, features):
        return 2 * -(-features // cls.GATE_BLOCK) * cls.GATE_BLOCK

    @classmethod
    def pair_gate_up(cls, w_gate, w_up):
        """The layout ``gated_gemm`` takes its weights in: blocks of 16 gate rows alternate with the 16 up
        rows of the same features; the feature count is padded to a multiple of 16 with zero rows.
        [..., N, K] twice -> [..., paired_rows(N), K]."""
        if w_gate.shape != w_up.shape:
            raise KernelError("pair_gate_up: gate and up weights differ in shape")
        *lead, n, k = w_gate.shape
        b = cls.GATE_BLOCK
        blocks = -(-n // b)
        out = w_gate.new_zeros((*lead, blocks, 2, b, k))
        flat = out.view(*lead, blocks, 2, b, k)
        pad = blocks * b - n
        for half, w in enumerate((w_gate, w_up)):
            if pad:
                w = torch.cat([w, w.new_zeros((*lead, pad, k))], -2)
            flat[..., half, :, :] = w.reshape(*lead, blocks, b, k)
        return out.view(*lead, 2 * blocks * b, k)

    def gated_gemm(self, x, w13, out, act="silu", plan: MoePlan | None = None, act_params=None):
        """out = act(x @ Wg.T) * (x @ Wu.T); w13 = pair_gate_up(Wg, Wu): [paired_rows(N), K], or with a
        plan (rows grouped by expert) [E, paired_rows(N), K].  act "swish_clamped" with act_params (slope, limit):
        g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(slope g) (u + 1); it runs as a plain
        product over the paired rows and an activation kernel over its float32 sums."""
        if act == "swish_clamped":
            if act_params is None or plan is not None:
                raise KernelError("gated_gemm: swish_clamped takes (slope, limit) and no plan")
            _check(out, "out", dims=2)
            M, N = out.shape
            if w13.dim() != 2 or w13.shape[0] != self.paired_rows(N) or w13.shape[1] != x.shape[1] or x.shape[0] != M:
                raise KernelError("gated_gemm: shapes do not match")
            parts = self.gemm_partials(x, w13)
            return self._run("elementwise", "flint_gated_act", _ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)),
                             _ptr(out), c_int(_code(out.dtype)), c_int(M), c_int(N), c_int(2), c_float(act_params[0]),
                             c_float(act_params[1]))
        self._gemm(x, w13, True, out, None, False, act, plan)

    ROW_ACTS = {"none": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "silu": 3, "relu2": 4}

    def row_act(self, partials, out, act, row_of=None, row_scale=None):
        """out[r] = act(scale_r * sum_z partials[z][r]): partials [S, rows, N] float32 (an ungated product left as
        partial sums).  With ``row_of`` [T, top] (the row of every (token, choice)) and ``row_scale`` [T, >= top], row
        row_of[t, c] is scaled by row_scale[t, c] before the activation; else every row by 1."""
        if partials.dim() == 2:
            partials = partials.unsqueeze(0)
        _check(partials, "partials", torch.float32, 3)
        _check(out, "out", dims=2)
        S, rows, N = partials.shape
        if tuple(out.shape) != (rows, N) or act not in self.ROW_ACTS:
            raise KernelError(f"row_act: output {tuple(out.shape)} or activation {act!r} does not fit")
        top = stride = 0
        n_launch = rows
        if row_of is not None:
            _check(row_of, "row_of", torch.int32, 2)
            _check(row_scale, "row_scale", torch.float32, 2)
            top, stride = row_of.shape[1], row_scale.stride(0)
            if row_of.numel() != rows or row_scale.shape[0] != row_of.shape[0] or row_scale.shape[1] < top:
                raise KernelError("row_act: the row list does not match the rows")
        self._run("elementwise", "flint_row_act", _ptr(partials), c_int(S), c_longlong(partials.stride(0)), _ptr(out),
                  c_int(_code(out.dtype)), c_int(n_launch), c_int(N), c_int(self.ROW_ACTS[act]), _ptr(row_of), _ptr(row_scale),
                  c_int(top), c_int(stride))

    def grouped_gemm(self, x, w, out, plan: MoePlan, plan_ready=False):
        """out[r] = x[r] @ w[expert of row r].T; w [E, N, K].  ``plan_ready``: another product over the same plan
        has run since the plan was made (the kernel may then read the plan before it waits for the kernel before
        it, and fetch its first weights meanwhile)."""
        self._gemm(x, w, False, out, None, False, "silu", plan, plan_ready=plan_ready)

    def gemm_partials(self, x, w, splits=None, plan: MoePlan | None = None, plan_ready=False):
        """x @ w.T left as S partial sums over pieces of the K range: float32 [S, M, N], no bias.
        The next kernel (rotary write, row norm, gated activation) adds them up; S is 1 when nothing
        was split.  With a plan, rows are grouped by expert and w is [E, N, K]."""
        _check(x, "x", dims=2)
        _check(w, "w")
        M, K = x.shape
        N = w.shape[-2]
        if w.shape[-1] != K or (plan is None) != (w.dim() == 2):
            raise KernelError("gemm_partials: shapes do not match")
        if not self.tensor_core_ok(x, w, plan):
            out = torch.empty((1, M, N), dtype=torch.float32, device=x.device)
            self._gemm_simt(x, w, False, out[0], None, False, 0, plan, M, N, K)
            return out
        kb = -(-K // 64)
        stream_k = 0
        if plan is None:
            bn, E = self.token_tile(M), 1
            splits = splits or self._k_splits(M, N, K, bn)
        else:
            bn, E = plan.tile_rows, plan.n_experts
            if splits is None and bn <= 128 and kb >= 2:
                # few rows per expert: how many tiles there are is known on the device only, so the kernel
                # cuts the K blocks of all tiles into equal runs itself; a tile gets at most `splits` pieces
                stream_k, splits = 1, min(12, kb)
            splits = splits or 1
        if not stream_k:
            kbps = -(-kb // splits)
            splits = -(-kb // kbps)
        out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        self._label = self._product_label(N, K, plan, False)
        self._run("gemm_tc", "flint_gemm_tc", _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(0), _ptr(None),
                  _ptr(out), c_int(F32), c_int(N), c_int(0), c_int(0), _ptr(plan.tile_expert if plan else None),
                  _ptr(plan.tile_row0 if plan else None), _ptr(plan.n_tiles if plan else None),
                  _ptr(plan.offsets if plan else None), c_int(plan.max_tiles if plan else 0), c_int(E), c_int(M),
                  c_int(N), c_int(K), c_int(bn), c_int(splits), _ptr(out), c_int(1), c_int(stream_k),
                  c_int(1 if plan_ready and plan is not None else 0), _ptr(self.tc_error))
        return out

    def _k_splits(self, M, N, K, bn):
        """Pieces of the K range so that a product with few tiles still fills the device."""
        tiles = -(-N // 128) * -(-M // bn)
        kb = -(-K // 64)
        if tiles >= self.sm_count or kb < 8:
            return 1
        # as many pieces as still fit one wave of resident blocks (three per SM with the 16-row token tile, whose
        # four stages take 72 KB, else two; a second, partial wave would cost as much as a full one: with the
        # 32-row tile counted at three, 17 to 32 rows ran 432 items on 296 places and a decode step took 1.5 % longer)
        return max(1, min(((3 if bn < 32 else 2) * self.sm_count) // tiles, kb // 4, 16))

    def _gemm(self, x, w, gated, out, bias, accumulate, act, plan, plan_ready=False):
        _check(x, "x", dims=2, contiguous=False)
        _check(out, "out", dims=2, contiguous=False)
        if x.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("gemm: rows must be contiguous")
        _check(w, "w")
        M, K = x.shape
        if plan is None:
            if w.dim() != 2:
                raise KernelError("gemm: dense weights must be [N, K]")
        elif w.dim() != 3 or w.shape[0] != plan.n_experts:
            raise KernelError("gemm: grouped weights must be [E, N, K]")
        N = out.shape[1] if gated else w.shape[-2]
        if gated and w.shape[-2] != self.paired_rows(N):
            raise KernelError(f"gemm: paired gate/up weights for {N} features have {self.paired_rows(N)} rows, "
                              f"not {w.shape[-2]}")
        if w.shape[-1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"gemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
        if bias is not None:
            _check(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError("gemm: bias length does not match")
        act_code = {"silu": 0, "gelu_pytorch_tanh": 1}[act]
        if self.tensor_core_ok(x, w, plan):
            if gated and M <= 128:
                # few rows: the product is bound by streaming the weights, and a gated tile cannot split
                # its K range; run it as a plain product over the paired rows, split over K, and apply
                # the activation to the summed partial tiles
                parts = self.gemm_partials(x, w, plan=plan)
                self._run("elementwise", "flint_gated_act", _ptr(parts), c_int(parts.shape[0]),
                          c_longlong(parts.stride(0)), _ptr(out), c_int(_code(out.dtype)), c_int(M), c_int(N),
                          c_int(act_code), c_float(0.0), c_float(0.0))
                return
            self._gemm_tc(x, w, gated, out, bias, accumulate, act_code, plan, M, N, K, plan_ready)
        else:
            self._gemm_simt(x, w, gated, out, bias, accumulate, act_code, plan, M, N, K)

    # bfloat16 x bfloat16 with 16-byte aligned rows goes to the tensor cores; everything else
    # (float32 operands: the true 32-bit path; odd K) to the float32 pipes
    def tensor_core_ok(self, x, w, plan=None):
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and (plan is None or plan.tile_rows in (16, 32, 64, 128, 256)))

    @staticmethod
    def token_tile(rows):
        for bn in (16, 32, 64, 128):
            if rows <= bn:
                return bn
        return 256

    def moe_tile_rows(self, n_tokens, n_experts, weight_dtype, top=2):
        """Row-tile size the plan should use for grouped products over these weights (``top`` choices a token)."""
        if weight_dtype != torch.bfloat16:
            return 64
        return self.token_tile(-(-top * n_tokens // n_experts))

    def _gemm_tc(self, x, w, gated, out, bias, accumulate, act_code, plan, M, N, K, plan_ready=False):
        if plan is not None:
            bn, splits, E = plan.tile_rows, 1, plan.n_experts
        else:
            E = 1
            bn = self.token_tile(M)
            splits = 1 if gated else self._k_splits(M, N, K, bn)
        partial = None
        if splits > 1:
            partial = torch.empty(splits * M * N, dtype=torch.float32, device=x.device)
        self._label = self._product_label(N, K, plan, gated)
        self._run("gemm_tc", "flint_gemm_tc", _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(1 if gated else 0), _ptr(bias),
                  _ptr(out), c_int(_code(out.dtype)), c_int(out.stride(0)), c_int(1 if accumulate else 0),
                  c_int(act_code), _ptr(plan.tile_expert if plan else None), _ptr(plan.tile_row0 if plan else None),
                  _ptr(plan.n_tiles if plan else None), _ptr(plan.offsets if plan else None),
                  c_int(plan.max_tiles if plan else 0), c_int(E), c_int(M), c_int(N), c_int(K), c_int(bn),
                  c_int(splits), _ptr(partial), c_int(0), c_int(0), c_int(1 if plan_ready and plan is not None else 0),
                  _ptr(self.tc_error))

    @staticmethod
    def _product_label(N, K, plan, gated):
        """How a profile lists a product: its weight shape, and whether it is gated or over experts."""
        return f"{N}x{K}" + (" gated" if gated else "") + (" experts" if plan is not None else "")

    def _gemm_simt(self, x, w, gated, out, bias, accumulate, act_code, plan, M, N, K):
        if plan is not None and plan.tile_rows > 64:
            raise KernelError("gemm_simt: the plan's row tiles must not exceed 64 rows")
        self._label = self._product_label(N, K, plan, gated)
        self._run("gemm_simt", "flint_gemm_simt", _ptr(x), c_int(_code(x.dtype)), c_int(x.stride(0)), _ptr(w),
                  c_int(1 if gated else 0), c_int(_code(w.dtype)), _ptr(bias), _ptr(out), c_int(_code(out.dtype)),
                  c_int(out.stride(0)), c_int(1 if accumulate else 0), c_int(act_code),
                  _ptr(plan.tile_expert if plan else None), _ptr(plan.tile_row0 if plan else None),
                  _ptr(plan.n_tiles if plan else None), _ptr(plan.offsets if plan else None),
                  c_int(plan.max_tiles if plan else 0), c_int(plan.tile_rows if plan else 0), c_int(M), c_int(N), c_int(K))

    # ------------------------------------------------------------------ attention
    def attention_plan(self, T, nq, nkv, span, hd=128, bf16=True, ragged=True):
        """Which kernel and how to split the key range so that the device is filled:
        (kernel, keys per split, splits).  Few rows (decode), bfloat16, head sizes up to 128: the
        TMA-fed tensor-core kernel, one warp per (row, kv head, split); few rows otherwise: one block
        each on the float32 pipes; many rows: the warp-per-row kernel."""
        g_chunks = -(-(nq // nkv) // 4)
        base = T * nkv * g_chunks
        span = max(span, 1)
        if T <= 256 and hd <= 128 and bf16:
            # tensor-core decode kernel fed by TMA: 8 query heads per warp, at most one wave of 8 warps
            # per SM (a second, nearly empty wave would cost as much as a full one), at least 64 keys per warp
            base8 = T * nkv * -(-(nq // nkv) // 8)
            if span > 64 and (ragged or base8 >= 256 or (base8 >= 24 and base8 * span >= 24 * 16384)):
                # rows of different lengths, or many rows: the kernel cuts the keys of all rows into equal runs
                # itself; the count is the most pieces one (row, kv head) may be cut into: enough for one wave
                # of 8 warps per SM.  (Few rows of about the same length are a little faster with the key
                # range of each row cut into the same number of pieces, below; but from three rows on and about
                # 48 k keys in all, splits in fours leave part of the device idle, and equal runs win: measured
                # at 8 kv heads, of a decode step: 8 rows of 6,144 keys -4 %, of 8,192 -6 %, of 65,536 -19 %;
                # 16 rows of 3,072 -4 %, of 4,096 -5 %; 4 rows of 16,384 -3 %, of 65,536 -10 %; 3 rows of 32,768
                # -4 %; below that line the plan below is the faster by 1 to 3 %, and for two rows at any length.)
                return "stream", span, self._stream_slices(base8)
            n = max(1, min(span // 64, 8 * self.sm_count // base8))
            keys = -(-(-(-span // n)) // 16) * 16
            n = -(-span // keys)
            if n > 4 and n % 4:
                # splits in fours: the four warps of a block then hold one row's splits and merge them themselves
                # (the kernel divides a row's keys evenly over the splits; the last one may stay empty)
                n = n // 4 * 4
                keys = -(-(-(-span // n)) // 16) * 16
            if n == 4 and keys >= 384:
                # 19 to 31 rows of many keys: there is room for four to seven splits a row, and four leave up to
                # half of the warps without work while the others walk 24 steps and more; equal runs fill the
                # device (2,048 keys: -10 % of a decode step at 20 rows, -8 % at 24, -4 % at 28, -2 % at 31;
                # with 512 keys four splits of 8 steps are the faster)
                return "stream", span, self._stream_slices(base8)
            return "tma", keys, n
        if T <= 256:
            n = max(1, min(-(-span // 128), -(-8 * self.sm_count // base)))
            keys = -(-(-(-span // n)) // 128) * 128
            return "block", keys, -(-span // keys)
        if base >= 2048 or span <= 64:
            return "warp", span, 1
        n = min(-(-span // 64), -(-2048 // base))
        keys = -(-(-(-span // n)) // 32) * 32
        return "warp", keys, -(-span // keys)

    def _stream_slices(self, items):
        """The most pieces the stream kernel may cut one (row, kv head) item into: enough for one wave of
        8 warps per SM over all items."""
        return max(2, min(64, -(-8 * self.sm_count // items) + 1))

    def attention(self, q, cache, step, out, nq, nkv, hd, window, scale, tiling=None):
        """Attention of all rows of a step: long portions on the tensor cores (bfloat16, head
        sizes up to 128), decoded tokens and short portions row by row.  ``tiling``: the step's rows cut into
        tiles of up to 128 rows (``engine.step.Tiling``); without one every row goes row by row."""
        P = cache.page_size
        tc = (tiling is not None and tiling.n_tiles > 0 and q.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
              and hd <= 128 and (64 % P == 0 or P % 64 == 0) and step.attention_splits is None)
        if not tc:
            return self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale,
                                        step.max_kv_len, splits=step.attention_splits,
                                        ragged=not step.even_lengths, fresh_keys=step.longest_entry)
        self.attention_prefill_tc(q, cache, tiling.tiles, tiling.n_tiles, out, nq, nkv, hd, window, scale)
        if tiling.n_other_rows:
            self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale, step.max_kv_len,
                                 rows=tiling.other_rows, fresh_keys=step.longest_entry)

    def rope_attention_decode(self, qkv, bias, cos, sin, rot, style, cache, step, out, nq, nkv, hd, window, scale):
        """The rotary write and the attention of a batch of decoded tokens in one launch: qkv [S, T, W] float32
        (partial sums of the q/k/v projection, bias apart) becomes q, the rows' new keys and values go into the
        cache pages, and every row attends over its request's keys.  Returns False, having launched nothing, when
        the batch is not of the kind this kernel takes (then the caller runs the two kernels one after the
        other): it takes bfloat16 caches and outputs, head sizes up to 128, the half-split rotation, and batches
        whose requests are about equally long."""
        T = qkv.shape[1]
        if (style != "half" or step.attention_splits is not None or out.dtype != torch.bfloat16
                or cache.k.dtype != torch.bfloat16 or hd > 128 or step.n_tokens != len(step.entries) or T != step.n_tokens):
            return False
        span = min(step.max_kv_len, window) if window else step.max_kv_len
        kernel, keys, n = self.attention_plan(T, nq, nkv, span, hd, True, not step.even_lengths)
        g_chunks = -(-(nq // nkv) // 8)
        if kernel != "tma" or T * nkv * g_chunks > self.attention_arrivals.numel():
            return False
        if n % 4:
            # splits in fours: the four warps of a block share the row's queries and its new key and value
            n = max(4, n // 4 * 4)
            keys = -(-(-(-max(span, 1) // n)) // 16) * 16
        _check(qkv, "qkv", torch.float32, 3)
        _check(out, "out", torch.bfloat16, 2)
        if qkv.shape[2] != (nq + 2 * nkv) * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("rope_attention_decode: widths do not match the head counts")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != qkv.shape[2]):
            raise KernelError("rope_attention_decode: bias must be float32 of the qkv width")
        if tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd) or tuple(cache.v.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("rope_attention_decode: cache pages do not match the head counts")
        if rot and cos.shape[1] * 2 != rot:
            raise KernelError("rope_attention_decode: table width must be rot/2")
        scratch = torch.empty(T * nq * n * (hd + 2), dtype=torch.float32, device=qkv.device)
        self._run("attention_tc", "flint_attention_decode_fused", _ptr(qkv), c_int(qkv.shape[0]), c_longlong(qkv.stride(0)),
                  _ptr(bias), _ptr(cos), _ptr(sin), c_int(rot), _ptr(cache.k), _ptr(cache.v), c_int(cache.k.shape[0]),
                  _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(cache.page_size), _ptr(step.pos),
                  _ptr(step.slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale),
                  c_int(keys), c_int(n), _ptr(scratch), _ptr(self.tc_error), _ptr(step.status),
                  _ptr(self.attention_arrivals), c_int(self.attention_arrivals.numel()))
        return True

    def attention_prefill_tc(self, q, cache, tiles, n_tiles, out, nq, nkv, hd, window, scale):
        _check(q, "q", torch.bfloat16, 2)
        _check(out, "out", torch.bfloat16, 2)
        _check(tiles, "tiles", torch.int32)
        T = q.shape[0]
        if q.shape[1] != nq * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("attention_prefill_tc: q/out width does not match the head counts")
        if cache.k.dtype != torch.bfloat16 or tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("attention_prefill_tc: cache pages must be bfloat16 [page, kv head, P, head size]")
        self._run("attention_tc", "flint_attention_prefill_tc", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                  c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                  c_int(cache.page_size), _ptr(tiles), c_int(n_tiles), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                  c_int(hd), c_int(window), c_float(scale), _ptr(self.tc_error))

    def paged_attention(self, q, cache, pos, slot, out, nq, nkv, hd, window, scale, max_kv_len, splits=None,
                        kernel=None, rows=None, ragged=True, merge_in_kernel=True, fresh_keys=1 << 30):
        """rows: int32 list of the batch rows to compute (default: all).  ragged: the rows' key ranges may
        differ much in length (False: a decode batch whose requests are about equally long).
        merge_in_kernel (the tensor-core decode kernel with splits in fours): the pieces of a row's key range
        are merged by the block that finishes last; False: by a kernel of its own.
        fresh_keys: how many of a row's newest keys the kernel before this one in the stream may have written
        (1 for a batch of decoded tokens); the default assumes all of them."""
        _check(q, "q", dims=2)
        _check(out, "out", q.dtype, 2)
        T = q.shape[0]
        if q.shape[1] != nq * hd or tuple(out.shape) != (T, nq * hd):
            raise KernelError("paged_attention: q/out width does not match the head counts")
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
            T = rows.numel()
        if tuple(cache.k.shape[1:]) != (nkv, cache.page_size, hd):
            raise KernelError("paged_attention: cache pages do not match the head counts")
        span = min(max_kv_len, window) if window else max_kv_len
        auto_kernel, split_keys, n_splits = self.attention_plan(
            T, nq, nkv, span, hd, q.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16, ragged)
        kernel = kernel or auto_kernel
        if splits is not None:
            split_keys, n_splits = splits
            if kernel == "stream":          # a given split is kept: the kernel with fixed key ranges
                kernel = "tma"
        if split_keys * n_splits < span:
            raise KernelError(f"paged_attention: {n_splits} splits of {split_keys} keys do not cover {span} keys")
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(T * nq * n_splits * (hd + 2), dtype=torch.float32, device=q.device)
        arrivals = self.attention_arrivals if merge_in_kernel else None
        if kernel == "stream":
            if auto_kernel != "stream":
                n_splits = self._stream_slices(T * nkv * -(-(nq // nkv) // 8))
                scratch = torch.empty(T * nq * n_splits * (hd + 2), dtype=torch.float32, device=q.device)
            return self._run("attention_tc", "flint_attention_decode_stream", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                             c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                             c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                             c_int(hd), c_int(window), c_float(scale), c_int(n_splits), _ptr(scratch), _ptr(rows),
                             _ptr(self.tc_error), c_int(max(1, int(fresh_keys))))
        if kernel == "tma":
            if rows is not None and rows.numel() != T:
                raise KernelError("paged_attention: bad row list")
            return self._run("attention_tc", "flint_attention_decode_tc", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                             c_int(cache.k.shape[0]), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                             c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv),
                             c_int(hd), c_int(window), c_float(scale), c_int(split_keys), c_int(n_splits),
                             _ptr(scratch), _ptr(rows), _ptr(self.tc_error), _ptr(arrivals),
                             c_int(arrivals.numel() if arrivals is not None else 0), c_int(max(1, int(fresh_keys))))
        fn = {"warp": "flint_paged_attention", "block": "flint_paged_attention_block"}[kernel]
        self._run("attention", fn, _ptr(q), c_int(_code(q.dtype)), _ptr(cache.k), _ptr(cache.v),
                  c_int(_code(cache.k.dtype)), _ptr(cache.block_table), c_int(cache.block_table.shape[1]),
                  c_int(cache.page_size), _ptr(pos), _ptr(slot), _ptr(out), c_int(_code(out.dtype)), c_int(T),
                  c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(split_keys), c_int(n_splits),
                  _ptr(scratch), _ptr(rows))

    # ------------------------------------------------------------------ attention with kept first tokens and a sink
    def qkv_write(self, qkv, bias, pos, slot, cos, sin, rot, style, q_out, cache, nq, nkv, hd, vd, status,
                  v_keep=None, v_from=None, blend=0.0):
        """qkv [S, T, W] float32 (partial sums of the q/k/v projection, W = (nq + nkv) hd + nkv vd) plus ``bias``:
        q (the leading ``rot`` dims of every head rotated by the row's position) goes to q_out [T, nq hd], keys
        (rotated alike) and values into the row's cache page.  ``v_keep`` [T, nkv vd] float32 receives the values
        as projected; with ``v_from`` (same shape) the cached values are (1 - blend) v + blend v_from."""
        if style not in ("half", "interleaved"):
            raise KernelError(f"qkv_write: unknown rotation style {style!r}")
        if qkv.dim() == 2:
            qkv = qkv.unsqueeze(0)
        _check(qkv, "qkv", torch.float32, 3)
        S, T, W = qkv.shape
        if W != (nq + nkv) * hd + nkv * vd:
            raise KernelError("qkv_write: the projection's width does not match the head counts")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != W):
            raise KernelError("qkv_write: bias must be float32 of the projection's width")
        _check(q_out, "q_out", dims=2)
        if tuple(q_out.shape) != (T, nq * hd):
            raise KernelError(f"qkv_write: q_out must be [{T}, {nq * hd}]")
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if rot and cos.shape[1] * 2 != rot:
            raise KernelError("qkv_write: table width must be rot/2")
        k, v, bt, P = cache.k, cache.v, cache.block_table, cache.page_size
        if tuple(k.shape[1:]) != (nkv, P, hd) or tuple(v.shape[1:]) != (nkv, P, vd) or v.dtype != k.dtype:
            raise KernelError(f"qkv_write: cache pages are {tuple(k.shape[1:])} and {tuple(v.shape[1:])}, expected "
                              f"{(nkv, P, hd)} and {(nkv, P, vd)}")
        for name, t in (("v_keep", v_keep), ("v_from", v_from)):
            if t is not None:
                _check(t, name, torch.float32, 2)
                if tuple(t.shape) != (T, nkv * vd):
                    raise KernelError(f"qkv_write: {name} must be [{T}, {nkv * vd}]")
        self._run("attention_sink", "flint_qkv_write", _ptr(qkv), c_int(S), c_longlong(qkv.stride(0)), _ptr(bias), _ptr(pos),
                  _ptr(slot), _ptr(cos), _ptr(sin), c_int(rot), c_int(1 if style == "interleaved" else 0), _ptr(q_out),
                  c_int(_code(q_out.dtype)), _ptr(k), _ptr(v), c_int(_code(k.dtype)), _ptr(bt), c_int(bt.shape[1]), c_int(P),
                  c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(vd), _ptr(v_keep), _ptr(v_from), c_float(blend),
                  _ptr(status))

    def sink_attention_plan(self, T, nq, nkv, span):
        """(keys per split, splits): enough warps to fill the device, at least 64 keys each."""
        base = T * nkv * -(-(nq // nkv) // 4)
        span = max(span, 1)
        n = max(1, min(-(-span // 64), -(-8 * self.sm_count // base)))
        keys = -(-(-(-span // n)) // 32) * 32
        return keys, -(-span // keys)

    def sink_attention(self, q, cache, step, out, nq, nkv, hd, vd, window, keep_first, sinks, scale, splits=None,
                       tiling=None, rows=None, chunk=0, pool=0, sigmoid=None):
        """Every row over its request's cached keys [.., hd] and values [.., vd]: row at position p sees key j if
        j <= p and (p - j < window or j < keep_first) (window 0: all); ``sinks`` [nq] float32 (or None): a logit
        per query head that joins the softmax's denominator.  q [T, nq hd] -> out [T, nq vd].  ``tiling``: the step's
        rows cut into tiles of up to 64 rows (``engine.step.Tiling``): in bfloat16, with head sizes in multiples of
        16 up to 128, the tiles run on the tensor cores and only the rows in no tile row by row.  ``rows``: int32
        list of the batch rows to compute (default: all).  ``chunk`` c > 0 (instead of a window): the row sees key j
        if j <= p and floor(j / c) = floor(p / c).  ``pool`` P > 0 (with a window): behind the window the row also sees
        one mean key and value per block of P positions that lies wholly before it, from ``cache.pool_k`` /
        ``cache.pool_v`` (written by ``pool_write``), in the same softmax.  ``sigmoid`` = (cap, r1, r2, bias) instead
        of a softmax: key j weighs sigmoid(cap tanh(score / cap) - r1_h ln(1 + r2_h (p - j)) + bias_h), not normalised
        (cap 0: no cap; r1, r2, bias float32 [nq] or None)."""
        _check(q, "q", dims=2)
        _check(out, "out", q.dtype, 2)
        cap, r1, r2, w_bias = sigmoid if sigmoid is not None else (0.0, None, None, None)
        kind = "sigmoid" if sigmoid is not None else ("pooled" if pool else "softmax")     # profiles list the launches by it
        for name, t in (("r1", r1), ("r2", r2), ("bias", w_bias)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != nq):
                raise KernelError(f"sink_attention: {name} must be float32 [{nq}]")
        if pool and (not window or cache.pool_k is None or cache.pool_slots * pool < cache.page_size):
            raise KernelError("sink_attention: block means need a window and the cache's storage for them")
        T = q.shape[0]
        P = cache.page_size
        if chunk and (window or keep_first):
            raise KernelError("sink_attention: runs of a fixed length exclude a window and kept first tokens")
        if q.shape[1] != nq * hd or tuple(out.shape) != (T, nq * vd):
            raise KernelError("sink_attention: q/out width does not match the head counts")
        if tuple(cache.k.shape[1:]) != (nkv, P, hd) or tuple(cache.v.shape[1:]) != (nkv, P, vd):
            raise KernelError("sink_attention: cache pages do not match the head counts")
        if sinks is not None:
            _check(sinks, "sinks", torch.float32, 1)
            if sinks.numel() != nq:
                raise KernelError(f"sink_attention: sinks must have {nq} entries")
        if (tiling is not None and tiling.n_tiles > 0 and rows is None and splits is None
                and self.sink_attention_tiles_ok(q.dtype, cache.k.dtype, hd, vd)):
            _check(tiling.tiles, "tiles", torch.int32)
            self._label = kind
            self._run("attention_sink", "flint_sink_attention_tiles", _ptr(q), _ptr(cache.k), _ptr(cache.v),
                      _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(P), _ptr(tiling.tiles),
                      c_int(tiling.n_tiles), _ptr(out), c_int(nq), c_int(nkv), c_int(hd), c_int(vd), c_int(window),
                      c_int(keep_first), c_int(chunk), _ptr(sinks), c_float(scale), _ptr(cache.pool_k if pool else None),
                      _ptr(cache.pool_v if pool else None), c_int(pool), c_int(cache.pool_slots if pool else 0),
                      c_int(1 if sigmoid is not None else 0), c_float(cap), _ptr(r1), _ptr(r2), _ptr(w_bias))
            if not tiling.n_other_rows:
                return
            rows = tiling.other_rows
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
            T = rows.numel()
        span = min(step.max_kv_len, window + keep_first) if window else step.max_kv_len
        if pool:
            span = min(step.max_kv_len, window + step.max_kv_len // pool)
        if chunk:
            span = min(span, chunk)
        keys, n = splits if splits is not None else self.sink_attention_plan(T, nq, nkv, span)
        if keys * n < span:
            raise KernelError(f"sink_attention: {n} splits of {keys} keys do not cover {span} keys")
        scratch = torch.empty(T * nq * n * (vd + 2), dtype=torch.float32, device=q.device) if n > 1 else None
        self._label = kind
        self._run("attention_sink", "flint_sink_attention", _ptr(q), c_int(_code(q.dtype)), _ptr(cache.k), _ptr(cache.v),
                  c_int(_code(cache.k.dtype)), _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(P),
                  _ptr(step.pos), _ptr(step.slot), _ptr(out), c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(vd),
                  c_int(window), c_int(keep_first), c_int(chunk), _ptr(sinks), c_float(scale), c_int(keys), c_int(n),
                  _ptr(scratch), _ptr(rows), _ptr(cache.pool_k if pool else None), _ptr(cache.pool_v if pool else None),
                  c_int(pool), c_int(cache.pool_slots if pool else 0), c_int(1 if sigmoid is not None else 0), c_float(cap),
                  _ptr(r1), _ptr(r2), _ptr(w_bias))

    def pool_write(self, cache, step, nkv, hd, vd, pool):
        """Every row of the step whose position ends a block of ``pool`` positions writes the block's mean key and
        value (over the cache rows as they stand, float32 sums in the order of the positions) into ``cache.pool_k`` /
        ``cache.pool_v`` [page, kv head, means a page, width]: block b of a request lies in slot b % n of the request's
        page b // n, n = ``cache.pool_slots``."""
        if cache.pool_k is None or cache.pool_slots * pool < cache.page_size:
            raise KernelError("pool_write: the cache has no storage for block means of this size")
        P, E = cache.page_size, cache.pool_slots
        if tuple(cache.pool_k.shape[1:]) != (nkv, E, hd) or tuple(cache.pool_v.shape[1:]) != (nkv, E, vd):
            raise KernelError("pool_write: the block means' storage does not match the head counts")
        self._run("attention_sink", "flint_pool_write", _ptr(cache.k), _ptr(cache.v), _ptr(cache.pool_k), _ptr(cache.pool_v),
                  c_int(_code(cache.k.dtype)), _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(P),
                  _ptr(step.pos), _ptr(step.slot), c_int(step.n_tokens), c_int(nkv), c_int(hd), c_int(vd), c_int(pool),
                  c_int(E), _ptr(step.status))

    @staticmethod
    def sink_attention_tiles_ok(q_dtype, cache_dtype, hd, vd):
        """Whether tiles of rows can run on the tensor cores: bfloat16 rows and cache, head sizes in multiples of 16
        up to 128."""
        return (q_dtype == torch.bfloat16 and cache_dtype == torch.bfloat16 and hd % 16 == 0 and vd % 16 == 0
                and 16 <= hd <= 128 and 16 <= vd <= 128)

    # ------------------------------------------------------------------ matrix memory (mLSTM)
    def mlstm_scan(self, proj, b_gates, slot, seq_start, n_seq, state, out, H, D, V, cap):
        """proj [S, T, N] float32: partial sums of the projection [q | k | v | g | z_i | z_f] (N = 2 H D + 2 H V +
        2 H); b_gates [2 H]: the gates' biases.  Runs the recurrence over every request's rows in order (request e
        owns rows seq_start[e] .. seq_start[e + 1] - 1; ``seq_start`` None: row e alone), from and into ``state``
        [slots, H (D V + D + 1)] float32, and writes the heads' unnormalised outputs to out [T, H V] float32.
        Returns the output gate's pre-activations, a [T, H V] view."""
        if proj.dim() == 2:
            proj = proj.unsqueeze(0)
        _check(proj, "proj", torch.float32, 3)
        S, T, N = proj.shape
        if N != 2 * H * D + 2 * H * V + 2 * H:
            raise KernelError("mlstm_scan: the projection's width does not match the sizes")
        _check(b_gates, "b_gates", torch.float32, 1)
        _check(state, "state", torch.float32, 2)
        _check(out, "out", torch.float32, 2)
        if b_gates.numel() != 2 * H or tuple(out.shape) != (T, H * V) or state.shape[1] < H * (D * V + D + 1):
            raise KernelError("mlstm_scan: shapes do not match")
        if seq_start is not None:
            _check(seq_start, "seq_start", torch.int32, 1)
            if seq_start.numel() != n_seq + 1:
                raise KernelError("mlstm_scan: seq_start must have one entry more than there are requests")
        elif n_seq != T:
            raise KernelError("mlstm_scan: without seq_start every request brings one row")
        x = torch.empty((T, N), dtype=torch.float32, device=proj.device)
        self._run("mlstm", "flint_mlstm_prepare", _ptr(proj), c_int(S), c_longlong(proj.stride(0)), _ptr(b_gates), _ptr(x),
                  c_int(T), c_int(H), c_int(D), c_int(V), c_float(cap))
        coef = torch.empty((T, H, 4), dtype=torch.float32, device=proj.device)
        self._run("mlstm", "flint_mlstm_scan", _ptr(x), _ptr(slot), _ptr(seq_start), c_int(n_seq), _ptr(state),
                  c_longlong(state.stride(0)), _ptr(coef), _ptr(out), c_int(T), c_int(H), c_int(D), c_int(V))
        g0 = 2 * H * D + H * V
        return x[:, g0:g0 + H * V]

    def mlstm_finish(self, o, gate, norm_w, eps, out, H, V):
        """out[t, h] = o[t, h] / rms(o[t, h]) * norm_w[h] * sigmoid(gate[t, h]): o [T, H V] float32, gate a
        [T, H V] float32 view (rows may be strided), norm_w [H V] float32."""
        _check(o, "o", torch.float32, 2)
        _check(gate, "gate", torch.float32, 2, contiguous=False)
        _check(norm_w, "norm_w", torch.float32, 1)
        _check(out, "out", dims=2)
        T = o.shape[0]
        if o.shape[1] != H * V or tuple(gate.shape) != (T, H * V) or gate.stride(1) != 1 or norm_w.numel() != H * V \
                or tuple(out.shape) != (T, H * V):
            raise KernelError("mlstm_finish: shapes do not match")
        self._run("mlstm", "flint_mlstm_finish", _ptr(o), _ptr(gate), c_longlong(gate.stride(0)), _ptr(norm_w), c_float(eps),
                  _ptr(out), c_int(_code(out.dtype)), c_int(T), c_int(H), c_int(V))

    # ------------------------------------------------------------------ state carried from token to token
    def short_conv(self, u, col0, w, bias, act, pos, slot, state, y):
        """y[t, c] = act(bias[c] + sum_j w[c, j] u[t - taps + 1 + j, col0 + c]) over the rows of each request, zeros
        before its start: u [T, >= col0 + C] float32 rows (a view; rows may be strided), w [C, taps], y [T, C] float32.
        ``state`` [slots, >= (taps - 1) C] float32 (a view of the slab's rows) holds each request's last taps - 1
        inputs and is brought up to date.  act: "none" or "silu"."""
        _check(u, "u", torch.float32, 2, contiguous=False)
        _check(w, "w", torch.float32, 2)
        _check(y, "y", torch.float32, 2)
        C, taps = w.shape
        T = u.shape[0]
        if u.stride(1) != 1 or u.shape[1] < col0 + C or tuple(y.shape) != (T, C):
            raise KernelError("short_conv: shapes do not match")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != C):
            raise KernelError("short_conv: bias must be float32, one per channel")
        if act not in ("none", "silu"):
            raise KernelError(f"short_conv: unknown activation {act!r}")
        if taps > 1:
            if state is None:
                raise KernelError("short_conv: a convolution over time needs the requests' state")
            _check(state, "state", torch.float32, 2, contiguous=False)
            if state.stride(1) != 1 or state.shape[1] < (taps - 1) * C:
                raise KernelError("short_conv: the state's rows are too short")
        self._run("recurrent", "flint_short_conv", _ptr(u), c_longlong(u.stride(0)), c_int(col0), _ptr(w), _ptr(bias),
                  c_int(1 if act == "silu" else 0), _ptr(pos), _ptr(slot), _ptr(state),
                  c_longlong(state.stride(0) if state is not None else 0), _ptr(y), c_int(T), c_int(C), c_int(taps))
        self.launches += 1 if taps > 1 else 0

    def delta_prepare(self, y, b, a, dt_bias, a_log, qk, decay, beta, H, G, D, unit_eps):
        """Operands of the gated delta rule from y [T, 2 G D + H V] (q | k | v after their convolution): qk [T, 2 G D]
        = q and k as unit vectors per head (x / sqrt(sum x^2 + unit_eps); q also times D^(-1/2)); beta [T, H] =
        sigmoid(b) (b a [T, H] view); decay [T, H D] = exp(-exp(a_log[h]) softplus(a + dt_bias))."""
        _check(y, "y", torch.float32, 2)
        _check(b, "b", torch.float32, 2, contiguous=False)
        for name, t in (("a", a), ("qk", qk), ("decay", decay), ("beta", beta)):
            _check(t, name, torch.float32, 2)
        T = y.shape[0]
        if y.shape[1] < 2 * G * D or tuple(b.shape) != (T, H) or b.stride(1) != 1 or tuple(a.shape) != (T, H * D) \
                or tuple(qk.shape) != (T, 2 * G * D) or tuple(decay.shape) != (T, H * D) or tuple(beta.shape) != (T, H) \
                or dt_bias.numel() != H * D or a_log.numel() != H:
            raise KernelError("delta_prepare: shapes do not match")
        self._run("recurrent", "flint_delta_prepare", _ptr(y), c_longlong(y.stride(0)), _ptr(b), c_longlong(b.stride(0)),
                  _ptr(a), _ptr(dt_bias), _ptr(a_log), _ptr(qk), _ptr(decay), _ptr(beta), c_int(T), c_int(H), c_int(G),
                  c_int(D), c_float(unit_eps))

    def ssd_prepare(self, raw, dt_bias, a_log, dt, decay):
        """dt = softplus(raw + dt_bias), decay = exp(-exp(a_log) dt): raw a [T, H] float32 view, dt and decay [T, H]."""
        _check(raw, "raw", torch.float32, 2, contiguous=False)
        _check(dt, "dt", torch.float32, 2)
        _check(decay, "decay", torch.float32, 2)
        T, H = raw.shape
        if raw.stride(1) != 1 or tuple(dt.shape) != (T, H) or tuple(decay.shape) != (T, H) or dt_bias.numel() != H \
                or a_log.numel() != H:
            raise KernelError("ssd_prepare: shapes do not match")
        self._run("recurrent", "flint_ssd_prepare", _ptr(raw), c_longlong(raw.stride(0)), _ptr(dt_bias), _ptr(a_log), _ptr(dt),
                  _ptr(decay), c_int(T), c_int(H))

    def recurrence_scan(self, q, k, v, decay, delta, beta, dt, skip, slot, seq_start, n_seq, state, out, H, G, D, V):
        """Walks every request's rows in order (request e owns rows seq_start[e] .. seq_start[e + 1] - 1;
        ``seq_start`` None: row e alone) from and into ``state`` [slots, >= H D V] float32, per head a matrix S [D, V]:
        ``delta``: S <- diag(decay_t) S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t (decay [T, H D]);
        else:      S <- decay_t S + k_t (dt_t v_t)^T; o_t = S^T q_t + skip v_t (decay, dt [T, H]; skip [H] or None).
        q, k [T, G D] and v [T, H V] are float32 views (rows may be strided); out [T, H V] float32."""
        for name, t in (("q", q), ("k", k), ("v", v)):
            _check(t, name, torch.float32, 2, contiguous=False)
            if t.stride(1) != 1:
                raise KernelError(f"recurrence_scan: {name}'s rows must be dense")
        w1 = beta if delta else dt
        for name, t in (("decay", decay), ("beta" if delta else "dt", w1), ("out", out)):
            _check(t, name, torch.float32, 2)
        _check(state, "state", torch.float32, 2, contiguous=False)
        T = q.shape[0]
        if tuple(q.shape) != (T, G * D) or tuple(k.shape) != (T, G * D) or tuple(v.shape) != (T, H * V) \
                or tuple(decay.shape) != (T, H * D if delta else H) or tuple(w1.shape) != (T, H) \
                or tuple(out.shape) != (T, H * V) or state.stride(1) != 1 or state.shape[1] < H * D * V:
            raise KernelError("recurrence_scan: shapes do not match")
        if skip is not None and (skip.dtype != torch.float32 or skip.numel() != H):
            raise KernelError("recurrence_scan: skip must be float32, one per head")
        if seq_start is not None:
            _check(seq_start, "seq_start", torch.int32, 1)
            if seq_start.numel() != n_seq + 1:
                raise KernelError("recurrence_scan: seq_start must have one entry more than there are requests")
        elif n_seq != T:
            raise KernelError("recurrence_scan: without seq_start every request brings one row")
        self._label = f"{'delta' if delta else 'ssd'} H{H} D{D} V{V}"
        self._run("recurrent", "flint_recurrence_scan", _ptr(q), c_longlong(q.stride(0)), _ptr(k), c_longlong(k.stride(0)),
                  _ptr(v), c_longlong(v.stride(0)), _ptr(decay), c_int(1 if delta else 0), _ptr(w1), _ptr(skip), _ptr(slot),
                  _ptr(seq_start), c_int(n_seq), _ptr(state), c_longlong(state.stride(0)), _ptr(out), c_int(H), c_int(G),
                  c_int(D), c_int(V))

    def gated_norm(self, o, gate, gate_act, gate_first, w, eps, groups, out):
        """o [T, N] float32 in ``groups`` equal parts, each divided by its own root mean square (eps inside the
        root), times w (its numbers repeat over the row: one per dim of a head, or one per channel) and times
        act(gate) (a [T, N] float32 view; "sigmoid" or "silu"); ``gate_first``: the gate multiplies before the norm."""
        _check(o, "o", torch.float32, 2)
        _check(gate, "gate", torch.float32, 2, contiguous=False)
        _check(w, "w", torch.float32, 1)
        _check(out, "out", dims=2)
        T, N = o.shape
        if tuple(gate.shape) != (T, N) or gate.stride(1) != 1 or tuple(out.shape) != (T, N) or N % groups \
                or N % w.numel():
            raise KernelError("gated_norm: shapes do not match")
        if gate_act not in ("sigmoid", "silu"):
            raise KernelError(f"gated_norm: unknown gate {gate_act!r}")
        self._run("recurrent", "flint_gated_norm", _ptr(o), _ptr(gate), c_longlong(gate.stride(0)),
                  c_int(1 if gate_act == "silu" else 0), c_int(1 if gate_first else 0), _ptr(w), c_int(w.numel()), c_float(eps),
                  c_int(groups), c_int(N), _ptr(out), c_int(_code(out.dtype)), c_int(T))

    def branch_mean(self, branches, weights, eps, out):
        """out[t] = (1 / n) sum_b weights[b] * y_b[t] / sqrt(mean(y_b[t]^2) + eps), y_b the sum of branch b's partial
        sums plus its bias: ``branches`` [(partials [S, T, W] float32, bias [W] or None)], out [T, W] float32."""
        n = len(branches)
        if not 1 <= n <= 4 or len(weights) != n:
            raise KernelError("branch_mean: one to four branches, a weight each")
        _check(out, "out", torch.float32, 2)
        T, W = out.shape
        ptrs, strides, counts, biases, ws = [], [], [], [], []
        for (part, bias), w in zip(branches, weights):
            _check(part, "partials", torch.float32, 3)
            if tuple(part.shape[1:]) != (T, W) or w.dtype != torch.float32 or w.numel() != W:
                raise KernelError("branch_mean: shapes do not match")
            if bias is not None and (bias.dtype != torch.float32 or bias.numel() != W):
                raise KernelError("branch_mean: a bias must be float32 of the rows' width")
            ptrs.append(part.data_ptr())
            strides.append(part.stride(0))
            counts.append(part.shape[0])
            biases.append(bias.data_ptr() if bias is not None else 0)
            ws.append(w.data_ptr())
        arr = lambda ctype, vals: (ctype * n)(*vals)
        self._run("recurrent", "flint_branch_mean", c_int(n), arr(c_void_p, ptrs), arr(c_longlong, strides), arr(c_int, counts),
                  arr(c_void_p, biases), arr(c_void_p, ws), c_float(eps), _ptr(out), c_int(T), c_int(W))

    def post_norm(self, x, partials, bias, scale, residual_scale, gamma, beta, eps, mode, out_copy=None):
        """x <- norm(residual_scale x + scale * (sum of partials + bias)) in place: x [T, W] float32, partials
        [S, T, W] float32, scale [W] or None; ``mode`` "layer" or "rms"; ``out_copy`` [T, W] of another
        element type receives the result too."""
        _check(x, "x", torch.float32, 2)
        _check(partials, "partials", torch.float32, 3)
        T, W = x.shape
        if tuple(partials.shape[1:]) != (T, W) or gamma.numel() != W or gamma.dtype != torch.float32:
            raise KernelError("post_norm: shapes do not match")
        for name, t in (("bias", bias), ("scale", scale), ("beta", beta)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != W):
                raise KernelError(f"post_norm: {name} must be float32 of the rows' width")
        if out_copy is not None:
            _check(out_copy, "out_copy", dims=2)
            if tuple(out_copy.shape) != (T, W):
                raise KernelError("post_norm: the copy must have the rows' shape")
        self._run("recurrent", "flint_post_norm", _ptr(x), _ptr(partials), c_int(partials.shape[0]),
                  c_longlong(partials.stride(0)), _ptr(bias), _ptr(scale), c_float(residual_scale), _ptr(gamma), _ptr(beta),
                  c_float(eps), c_int({"layer": 0, "rms": 1}[mode]), _ptr(out_copy),
                  c_int(_code(out_copy.dtype) if out_copy is not None else F32), c_int(T), c_int(W))

    def depth_mix(self, history, n, w, h, out_copy=None):
        """history[n - 1] <- h, then h <- sum over j < n of w[j] history[j]: history [levels, T, W] float32, w [>= n]
        float32, h [T, W] float32; ``out_copy`` receives the new h in another element type too."""
        _check(history, "history", torch.float32, 3)
        _check(h, "h", torch.float32, 2)
        if n < 1 or n > history.shape[0] or tuple(history.shape[1:]) != tuple(h.shape) or w.numel() < n \
                or w.dtype != torch.float32:
            raise KernelError("depth_mix: shapes do not match")
        if out_copy is not None:
            _check(out_copy, "out_copy", dims=2)
        self._run("recurrent", "flint_depth_mix", _ptr(history), c_longlong(history.stride(0)), c_int(n), _ptr(w), _ptr(h),
                  _ptr(out_copy), c_int(_code(out_copy.dtype) if out_copy is not None else F32), c_longlong(h.numel()))

    def softcap(self, x, cap):
        """x <- cap tanh(x / cap) in place (float32)."""
        _check(x, "x", torch.float32)
        self._run("recurrent", "flint_softcap", _ptr(x), c_float(cap), c_longlong(x.numel()))

    def cast_rows(self, x, out):
        """out <- x in out's element type (x float32, same shape)."""
        _check(x, "x", torch.float32)
        _check(out, "out")
        if out.shape != x.shape:
            raise KernelError("cast_rows: shapes differ")
        self._run("recurrent", "flint_cast_rows", _ptr(x), _ptr(out), c_int(_code(out.dtype)), c_longlong(x.numel()))

    def qk_norm_write(self, y, q_norm, k_norm, eps, pos, slot, cos, sin, rot, style, v_cos, v_sin, v_style, q_out, cache,
                      nq, nkv, hd, vd, status, whole=False, v_from_k=False, q_temp=None):
        """y [T, (nq + nkv) hd + nkv vd] float32 (q | k | v): every q and k head is divided by its root mean square
        and scaled by q_norm / k_norm [hd] (both None: no norm), its leading ``rot`` dims rotate by the row's
        position; every value head rotates over all vd dims with tables of its own (None: not at all).  q goes to
        q_out [T, nq hd], keys and values into the row's cache page.  ``whole``: q is divided by one root mean square
        over all its heads and scaled by q_norm [nq hd], k likewise with k_norm [nkv hd].  ``v_from_k``: the values are
        the keys as projected, before norm and rotation (vd = hd; y has no value columns).  ``q_temp`` = (coef, every):
        q at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1)."""
        _check(y, "y", torch.float32, 2, contiguous=False)
        T = y.shape[0]
        if y.stride(1) != 1 or y.shape[1] < (nq + nkv) * hd + (0 if v_from_k else nkv * vd):
            raise KernelError("qk_norm_write: the rows' width does not match the head counts")
        if v_from_k and vd != hd:
            raise KernelError("qk_norm_write: values that are the keys need vd = hd")
        qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 1)
        _check(q_out, "q_out", dims=2)
        if tuple(q_out.shape) != (T, nq * hd):
            raise KernelError(f"qk_norm_write: q_out must be [{T}, {nq * hd}]")
        for name, t, n in (("q_norm", q_norm, nq * hd if whole else hd), ("k_norm", k_norm, nkv * hd if whole else hd)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != n):
                raise KernelError(f"qk_norm_write: {name} must be float32 [{n}]")
        if rot and (cos is None or cos.shape[1] * 2 != rot):
            raise KernelError("qk_norm_write: table width must be rot/2")
        if v_cos is not None and v_cos.shape[1] * 2 != vd:
            raise KernelError("qk_norm_write: the values' table width must be vd/2")
        k, v, bt, P = cache.k, cache.v, cache.block_table, cache.page_size
        if tuple(k.shape[1:]) != (nkv, P, hd) or tuple(v.shape[1:]) != (nkv, P, vd) or v.dtype != k.dtype:
            raise KernelError(f"qk_norm_write: cache pages are {tuple(k.shape[1:])} and {tuple(v.shape[1:])}, expected "
                              f"{(nkv, P, hd)} and {(nkv, P, vd)}")
        self._run("recurrent", "flint_qk_norm_write", _ptr(y), c_longlong(y.stride(0)), _ptr(q_norm), _ptr(k_norm), c_float(eps),
                  _ptr(pos), _ptr(slot), _ptr(cos), _ptr(sin), c_int(rot), c_int(1 if style == "interleaved" else 0),
                  _ptr(v_cos), _ptr(v_sin), c_int(1 if v_style == "interleaved" else 0), _ptr(q_out),
                  c_int(_code(q_out.dtype)), _ptr(k), _ptr(v), c_int(_code(k.dtype)), _ptr(bt), c_int(bt.shape[1]), c_int(P),
                  c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(vd), c_int(1 if whole else 0),
                  c_int(1 if v_from_k else 0), c_float(qt_coef), c_int(qt_every), _ptr(status))

    def head_finish(self, attn, pos, v_cos, v_sin, v_style, gate, out, nq, vd):
        """attn [T, nq vd]: every head's sum is turned back by the row's position (tables None: not at all) and
        multiplied by sigmoid(gate[t, head]) (gate a [T, nq] float32 view, or None), or, with a gate [T, nq vd], number
        by number by sigmoid(gate[t, head, d])."""
        _check(attn, "attn", dims=2)
        _check(out, "out", attn.dtype, 2)
        T = attn.shape[0]
        if tuple(attn.shape) != (T, nq * vd) or out.shape != attn.shape:
            raise KernelError("head_finish: shapes do not match")
        if gate is not None:
            _check(gate, "gate", torch.float32, 2, contiguous=False)
            if tuple(gate.shape) not in ((T, nq), (T, nq * vd)) or gate.stride(1) != 1:
                raise KernelError("head_finish: the gates must be [rows, heads] or [rows, heads x value dims]")
        self._run("recurrent", "flint_head_finish", _ptr(attn), c_int(_code(attn.dtype)), _ptr(pos), _ptr(v_cos), _ptr(v_sin),
                  c_int(1 if v_style == "interleaved" else 0), _ptr(gate),
                  c_longlong(gate.stride(0) if gate is not None else 0),
                  c_int(1 if gate is not None and gate.shape[1] == nq * vd and vd > 1 else 0), _ptr(out), c_int(T), c_int(nq),
                  c_int(vd))

    def sum_norm_add(self, dst, branches=(), scales=(), expert_rows=None, gamma=None, eps=0.0, accumulate=True):
        """r[t] = sum_b scales[b] * y_b[t] + sum_j gates[t, j] * y[row_of[t, j]] with y_b the sum of branch b's partial
        sums plus its bias (``branches`` [(partials [S, T, W] float32, bias [W] or None)], up to four) and
        ``expert_rows`` = (y [*, W], row_of [T, k] int32, gates [T, k]) or None; with ``gamma`` [W]:
        r <- r / sqrt(mean(r^2) + eps) * gamma; then dst [T, W] float32 += r (``accumulate``) or dst = r."""
        _check(dst, "dst", torch.float32, 2)
        T, W = dst.shape
        n = len(branches)
        if n > 4 or len(scales) != n:
            raise KernelError("sum_norm_add: up to four branches, a scale each")
        ptrs, strides, counts, biases = [], [], [], []
        for part, bias in branches:
            _check(part, "partials", torch.float32, 3)
            if tuple(part.shape[1:]) != (T, W):
                raise KernelError("sum_norm_add: shapes do not match")
            if bias is not None and (bias.dtype != torch.float32 or bias.numel() != W):
                raise KernelError("sum_norm_add: a bias must be float32 of the rows' width")
            ptrs.append(part.data_ptr())
            strides.append(part.stride(0))
            counts.append(part.shape[0])
            biases.append(bias.data_ptr() if bias is not None else 0)
        y = row_of = gates = None
        k = 0
        if expert_rows is not None:
            y, row_of, gates = expert_rows
            _check(y, "y", torch.float32, 2)
            _check(row_of, "row_of", torch.int32, 2)
            _check(gates, "gates", torch.float32, 2)
            k = row_of.shape[1]
            if y.shape[1] != W or tuple(row_of.shape) != (T, k) or tuple(gates.shape) != (T, k):
                raise KernelError("sum_norm_add: the expert rows' shapes do not match")
        if gamma is not None and (gamma.dtype != torch.float32 or gamma.numel() != W):
            raise KernelError("sum_norm_add: gamma must be float32 of the rows' width")
        m = max(n, 1)
        arr = lambda ctype, vals: (ctype * m)(*vals)
        self._run("recurrent", "flint_sum_norm_add", c_int(n), arr(c_void_p, ptrs), arr(c_longlong, strides), arr(c_int, counts),
                  arr(c_void_p, biases), arr(c_float, [float(x) for x in scales]), _ptr(y), _ptr(row_of), _ptr(gates), c_int(k),
                  _ptr(gamma), c_float(eps), _ptr(dst), c_int(1 if accumulate else 0), c_int(T), c_int(W))

    def retention_prepare(self, proj, pos, cos, sin, rot, style, decay_h, dt_value, qk, decay, dt, H, D):
        """proj [T, >= 2 H D] float32 (q | k, H heads of D dims; rows may be strided): the leading ``rot`` dims of
        every head turn by the row's position into qk [T, 2 H D]; decay [T, H] <- decay_h [H] and dt [T, H] <- dt_value
        on every row (what the recurrence kernel takes per token)."""
        _check(proj, "proj", torch.float32, 2, contiguous=False)
        T = proj.shape[0]
        if proj.stride(1) != 1 or proj.shape[1] < 2 * H * D:
            raise KernelError("retention_prepare: the rows do not hold q and k")
        for name, t, shape in (("qk", qk, (T, 2 * H * D)), ("decay", decay, (T, H)), ("dt", dt, (T, H))):
            _check(t, name, torch.float32, 2)
            if tuple(t.shape) != shape:
                raise KernelError(f"retention_prepare: {name} must be {shape}")
        if decay_h.dtype != torch.float32 or decay_h.numel() != H:
            raise KernelError("retention_prepare: one float32 decay per head")
        if rot and (cos is None or cos.shape[1] * 2 != rot):
            raise KernelError("retention_prepare: table width must be rot/2")
        self._run("recurrent", "flint_retention_prepare", _ptr(proj), c_longlong(proj.stride(0)), _ptr(pos), _ptr(cos),
                  _ptr(sin), c_int(rot), c_int(1 if style == "interleaved" else 0), _ptr(decay_h), c_float(dt_value), _ptr(qk),
                  _ptr(decay), _ptr(dt), c_int(T), c_int(H), c_int(D))

    # ------------------------------------------------------------------ attention over a cached latent
    def head_products(self, x, w, out):
        """A small product per head: out[t, h, :] = w[h] @ x[t, h, :].  x [T, H, K], w [H, N, K], out [T, H, N]; x and
        out may be views into wider rows (their last axis contiguous)."""
        _check(x, "x", dims=3, contiguous=False)
        _check(out, "out", dims=3, contiguous=False)
        _check(w, "w", dims=3)
        T, H, K = x.shape
        N = w.shape[1]
        if w.shape[0] != H or w.shape[2] != K or tuple(out.shape) != (T, H, N):
            raise KernelError(f"head_products: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
        if x.stride(2) != 1 or out.stride(2) != 1:
            raise KernelError("head_products: the last axis must be contiguous")
        if (x.dtype == w.dtype == out.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            # all heads in one launch on the tensor cores
            return self._run("latent", "flint_head_products", _ptr(x), c_longlong(x.stride(0)), c_longlong(x.stride(1)),
                             _ptr(w), _ptr(out), c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(T), c_int(H),
                             c_int(N), c_int(K))
        for h in range(H):
            self.gemm(x[:, h, :], w[h], out[:, h, :])

    def latent_prepare(self, proj, pos, slot, cos, sin, rot_dims, style, norm_w, eps, q_plain, qa, cache, H, D, R, C,
                       write_kv, status):
        """proj [S, T, W] float32 (partial sums of [q | latent] projections, W = H (D + R) + (C + R if
        ``write_kv``)): the plain q dims go to q_plain [T, H, D], the rotated q dims into the last R numbers of
        qa [T, H, C + R], and, with ``write_kv``, the token's cache row [normed latent | rotated key part | 0...]
        into its page.  ``rot_dims`` of the R dims rotate, in ``style`` ("interleaved": 2i with 2i + 1;
        "half": i with i + rot_dims/2)."""
        if style not in ("half", "interleaved"):
            raise KernelError(f"latent_prepare: unknown rotation style {style!r}")
        if proj.dim() == 2:
            proj = proj.unsqueeze(0)
        _check(proj, "proj", torch.float32, 3)
        S, T, W = proj.shape
        if W != H * (D + R) + ((C + R) if write_kv else 0):
            raise KernelError("latent_prepare: the projection's width does not match the sizes")
        _check(q_plain, "q_plain", qa.dtype, 3)
        _check(qa, "qa", dims=3)
        if tuple(q_plain.shape) != (T, H, D) or tuple(qa.shape) != (T, H, C + R):
            raise KernelError("latent_prepare: q buffers do not match the sizes")
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if rot_dims and cos.shape[1] * 2 != rot_dims:
            raise KernelError("latent_prepare: table width must be rot_dims/2")
        k = bt = None
        cdt, P, max_pages, row_w = F32, 16, 0, 0
        if write_kv:
            k, bt, P = cache.k, cache.block_table, cache.page_size
            cdt, max_pages, row_w = _code(k.dtype), bt.shape[1], k.shape[-1]
            if tuple(k.shape[1:]) != (1, P, row_w) or row_w < C + R or row_w % 8:
                raise KernelError(f"latent_prepare: cache pages are {tuple(k.shape[1:])}, expected (1, {P}, >= {C + R})")
            if norm_w is None or norm_w.dtype != torch.float32 or norm_w.numel() != C:
                raise KernelError("latent_prepare: the latent's norm scale must be float32 of the latent size")
        self._run("latent", "flint_latent_prepare", _ptr(proj), c_int(S), c_longlong(proj.stride(0)), _ptr(pos), _ptr(slot),
                  _ptr(cos), _ptr(sin), c_int(rot_dims), c_int(1 if style == "interleaved" else 0), _ptr(norm_w),
                  c_float(eps), _ptr(q_plain), _ptr(qa), c_int(_code(qa.dtype)), _ptr(k), c_int(cdt), _ptr(bt),
                  c_int(max_pages), c_int(P), c_int(T), c_int(H), c_int(D), c_int(R), c_int(C), c_int(row_w),
                  c_int(1 if write_kv else 0), _ptr(status))

    def latent_attention_plan(self, T, H, span):
        """(keys per split, splits) for the float32-pipe kernel: enough warps to fill the device, at least 64
        keys each."""
        base = T * -(-H // 4)
        n = max(1, min(-(-max(span, 1) // 64), -(-8 * self.sm_count // base)))
        keys = -(-(-(-max(span, 1) // n)) // 32) * 32
        return keys, -(-max(span, 1) // keys)

    def latent_attention(self, qa, cache, step, out, H, C, window, scale, splits=None, rows=None, kernel=None):
        """Every row's heads over its request's cached latent rows: qa [T, H, Dk] (key up-projection folded in)
        -> out [T, H, C], the probability-weighted sum of the latents (causal, ``window`` 0 = all keys).
        bfloat16 rows run on the tensor cores (``kernel`` "mma"), everything else, and a list of ``rows``, on the
        float32 pipes ("simt")."""
        _check(qa, "qa", dims=3)
        _check(out, "out", qa.dtype, 3)
        T, Dk = qa.shape[0], qa.shape[2]
        k, P = cache.k, cache.page_size
        row_w = k.shape[-1]
        if qa.shape[1] != H or tuple(out.shape) != (T, H, C) or tuple(k.shape[1:]) != (1, P, row_w) or row_w < Dk:
            raise KernelError("latent_attention: shapes do not match")
        span = min(step.max_kv_len, window) if window else step.max_kv_len
        mma_ok = qa.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and rows is None and C <= 512 and row_w <= 640
        if kernel is None:
            kernel = "mma" if mma_ok else "simt"
        if kernel == "mma":
            if not mma_ok:
                raise KernelError("latent_attention: the tensor-core kernel takes bfloat16 rows of up to 512 latent dims, all rows")
            nh = min(H, 32)
            decode = T == len(getattr(step, "entries", ()))          # one token a request: a block per token
            nt = 1 if decode else max(1, 32 // nh)
            if splits is None:
                blocks = -(-T // nt) * -(-H // nh)
                n = max(1, min(-(-max(span, 1) // 128), (2 * self.sm_count) // blocks))
                keys = -(-(-(-max(span, 1) // n)) // 64) * 64
                splits = (keys, -(-max(span, 1) // keys))
            keys, n = splits
            if keys * n < span:
                raise KernelError(f"latent_attention: {n} splits of {keys} keys do not cover {span} keys")
            scratch = torch.empty(T * H * n * (C + 2), dtype=torch.float32, device=qa.device) if n > 1 else None
            return self._run("latent", "flint_latent_attention_mma", _ptr(qa), _ptr(k), _ptr(cache.block_table),
                             c_int(cache.block_table.shape[1]), c_int(P), _ptr(step.pos), _ptr(step.slot), _ptr(out),
                             c_int(T), c_int(H), c_int(C), c_int(Dk), c_int(row_w), c_int(window), c_float(scale),
                             c_int(nt), c_int(nh), c_int(keys), c_int(n), _ptr(scratch))
        if kernel != "simt":
            raise KernelError(f"latent_attention: unknown kernel {kernel!r}")
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
            T = rows.numel()
        keys, n = splits if splits is not None else self.latent_attention_plan(T, H, span)
        if keys * n < span:
            raise KernelError(f"latent_attention: {n} splits of {keys} keys do not cover {span} keys")
        scratch = torch.empty(T * H * n * (C + 2), dtype=torch.float32, device=qa.device) if n > 1 else None
        self._run("latent", "flint_latent_attention", _ptr(qa), c_int(_code(qa.dtype)), _ptr(k), c_int(_code(k.dtype)),
                  _ptr(cache.block_table), c_int(cache.block_table.shape[1]), c_int(P), _ptr(step.pos), _ptr(step.slot),
                  _ptr(out), c_int(T), c_int(H), c_int(C), c_int(Dk), c_int(row_w), c_int(window), c_float(scale),
                  c_int(keys), c_int(n), _ptr(scratch), _ptr(rows))

    # ------------------------------------------------------------------ additions to the embedded rows
    def pair_embed_add(self, ids, pos, slot, last, table, out, mul_prev, mul_cur, fed_rows=None, fed_from=None):
        """out [T, H] += table[row of the pair (previous token, token)]: row (prev * mul_prev + cur * mul_cur) mod
        buckets, table [buckets + 1, H] with the last row for a sequence's first token.  ``last`` [slots] int32
        holds each request's newest token between steps and is renewed here."""
        _check(ids, "ids", torch.int32, 1)
        _check(last, "last", torch.int32, 1)
        _check(table, "table", dims=2)
        _check(out, "out", torch.float32, 2)
        T, H = out.shape
        if ids.numel() != T or table.shape[1] != H or table.shape[0] < 2:
            raise KernelError("pair_embed_add: shapes do not match")
        if (fed_rows is None) != (fed_from is None):
            raise KernelError("pair_embed_add: fed rows and their source come together")
        pair_row = torch.empty(T, dtype=torch.int32, device=out.device)
        self._run("elementwise", "flint_pair_embed_add", _ptr(ids), _ptr(fed_rows), _ptr(fed_from), _ptr(pos), _ptr(slot),
                  _ptr(last), _ptr(pair_row), _ptr(table), c_int(_code(table.dtype)), _ptr(out), c_int(T), c_int(H),
                  c_longlong(int(mul_prev)), c_longlong(int(mul_cur)), c_int(table.shape[0] - 1))

    # ------------------------------------------------------------------ routing
    def router_sparsemixer(self, x, wr, eps, expert_ids, gates, logits_out=None):
        _check(x, "x", torch.float32, 2)
        _check(wr, "router weight", dims=2)
        T, H = x.shape
        E = wr.shape[0]
        if wr.shape[1] != H:
            raise KernelError("router: weight width does not match")
        _check(expert_ids, "expert_ids", torch.int32)
        _check(gates, "gates", torch.float32)
        self._run("moe", "flint_router_sparsemixer", _ptr(x), _ptr(wr), c_int(_code(wr.dtype)), c_float(eps),
                  _ptr(expert_ids), _ptr(gates), _ptr(logits_out), c_int(T), c_int(H), c_int(E))

    def route(self, x, router):
        """Serve a ``RouterRequest`` on normalised rows x [T, H] float32 with the stand-alone kernels."""
        if getattr(router, "rule", "") == "sigmoid":
            return self.router_sigmoid(x, router.weight, router.weight.shape[0] - router.extra, router.top, router.expert_ids,
                                       router.gates, router.weights, getattr(router, "logits", None))
        if getattr(router, "rule", "") == "sigmoid_grouped":
            return self.router_sigmoid_grouped(x, router.weight, router.correction, router.top, router.groups, router.keep,
                                               router.normalize, router.scale, router.expert_ids, router.gates,
                                               getattr(router, "logits", None))
        if int(getattr(router, "top", 0)) > 0:
            return self.router_topk(x, router.weight, router.top, router.groups, router.keep, router.scale,
                                    router.expert_ids, router.gates, getattr(router, "logits", None))
        return self.router_sparsemixer(x, router.weight, router.jitter_eps, router.expert_ids, router.gates,
                                       getattr(router, "logits", None))

    def router_topk(self, x, wr, top, n_groups, keep, scale, expert_ids, gates, logits_out=None):
        """Softmax router whose choice is limited to groups: scores softmax(x @ wr.T) in float32; the experts form
        ``n_groups`` equal groups of neighbours, a group scores as its best member, the ``top`` best experts of
        the ``keep`` best groups are chosen; gates are the chosen scores over their sum, times ``scale``.
        expert_ids and gates [T, top]."""
        _check(x, "x", torch.float32, 2)
        _check(wr, "router weight", dims=2)
        T, H = x.shape
        E = wr.shape[0]
        if wr.shape[1] != H:
            raise KernelError("router: weight width does not match")
        _check(expert_ids, "expert_ids", torch.int32, 2)
        _check(gates, "gates", torch.float32, 2)
        if tuple(expert_ids.shape) != (T, top) or tuple(gates.shape) != (T, top):
            raise KernelError(f"router: choices and gates must be [{T}, {top}]")
        if logits_out is not None:
            _check(logits_out, "router logits", torch.float32, 2)
        self._run("moe", "flint_router_topk", _ptr(x), _ptr(wr), c_int(_code(wr.dtype)), c_int(top), c_int(n_groups),
                  c_int(keep), c_float(scale), _ptr(expert_ids), _ptr(gates), _ptr(logits_out), c_int(T), c_int(H), c_int(E))

    def router_sigmoid(self, x, wr, E, top, expert_ids, scores, weights, logits_out=None):
        """Sigmoid router: scores sigmoid(x @ wr[:E].T) in float32, the ``top`` largest chosen (the lower index among
        equals), expert_ids and scores [T, top].  Rows of wr beyond E are gates of always-on parts: weights
        [T, top + X] gets 1 for the chosen experts and the sigmoids of those rows after them."""
        _check(x, "x", torch.float32, 2)
        _check(wr, "router weight", dims=2)
        T, H = x.shape
        X = wr.shape[0] - E
        if wr.shape[1] != H or X < 0:
            raise KernelError("router: weight shape does not match")
        _check(expert_ids, "expert_ids", torch.int32, 2)
        _check(scores, "scores", torch.float32, 2)
        _check(weights, "weights", torch.float32, 2)
        if tuple(expert_ids.shape) != (T, top) or tuple(scores.shape) != (T, top) or tuple(weights.shape) != (T, top + X):
            raise KernelError(f"router: choices and scores must be [{T}, {top}], weights [{T}, {top + X}]")
        if logits_out is not None:
            _check(logits_out, "router logits", torch.float32, 2)
            if tuple(logits_out.shape) != (T, E + X):
                raise KernelError(f"router: logits must be [{T}, {E + X}]")
        self._run("moe", "flint_router_sigmoid", _ptr(x), _ptr(wr), c_int(_code(wr.dtype)), c_int(E), c_int(X), c_int(top),
                  _ptr(expert_ids), _ptr(scores), _ptr(weights), _ptr(logits_out), c_int(T), c_int(H))

    def router_sigmoid_grouped(self, x, wr, correction, top, n_groups, keep, normalize, scale, expert_ids, gates,
                               logits_out=None):
        """Scores sigmoid(x wr^T) in float32; choice scores add ``correction`` [E] (or None); a group of neighbouring
        experts scores as the sum of its two largest choice scores, only the ``keep`` best of ``n_groups`` groups may be
        chosen from, the ``top`` largest choice scores are (the lower index among equals); gates [T, top]: the chosen
        experts' scores, over their sum (+ 1e-20) if ``normalize``, times ``scale``."""
        _check(x, "x", torch.float32, 2)
        _check(wr, "router weight", dims=2)
        _check(expert_ids, "expert_ids", torch.int32, 2)
        _check(gates, "gates", torch.float32, 2)
        T, H = x.shape
        E = wr.shape[0]
        if wr.shape[1] != H or tuple(expert_ids.shape) != (T, top) or tuple(gates.shape) != (T, top):
            raise KernelError("router_sigmoid_grouped: shapes do not match")
        if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
            raise KernelError("router_sigmoid_grouped: the correction must be float32, one per expert")
        if logits_out is not None:
            _check(logits_out, "logits_out", torch.float32, 2)
        self._run("moe", "flint_router_sigmoid_grouped", _ptr(x), _ptr(wr), c_int(_code(wr.dtype)), _ptr(correction), c_int(E),
                  c_int(top), c_int(n_groups), c_int(keep), c_int(1 if normalize else 0), c_float(scale), _ptr(expert_ids),
                  _ptr(gates), _ptr(logits_out), c_int(T), c_int(H))

    def _plan_buffers(self, expert_ids, n_experts, tile_rows):
        _check(expert_ids, "expert_ids", torch.int32, 2)
        n, top = expert_ids.numel(), expert_ids.shape[1]
        dev = expert_ids.device
        max_tiles = n // tile_rows + min(n_experts, n)
        ints = torch.empty(n_experts + (n_experts + 1) + n + n + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
        o = 0
        parts = []
        for size in (n_experts, n_experts + 1, n, n, max_tiles, max_tiles, 1):
            parts.append(ints[o:o + size])
            o += size
        counts, offsets, row_of, token_of, tile_expert, tile_row0, n_tiles = parts
        plan = MoePlan(n_experts, tile_rows, max_tiles, counts, offsets, row_of.view(-1, top), token_of,
                       tile_expert, tile_row0, n_tiles, top)
        return plan, [_ptr(t) for t in parts]

    def moe_plan(self, expert_ids, n_experts, tile_rows) -> MoePlan:
        plan, ptrs = self._plan_buffers(expert_ids, n_experts, tile_rows)
        self._run("moe", "flint_moe_plan", _ptr(expert_ids), c_int(expert_ids.numel()), c_int(n_experts),
                  c_int(tile_rows), *ptrs, c_int(plan.max_tiles), c_int(plan.top))
        return plan

    def moe_dispatch(self, expert_ids, n_experts, tile_rows, x):
        """The plan for these choices and the rows of x in its order: (plan, xs) with
        xs[r] = x[plan.token_of[r]].  Few rows take one fused launch."""
        _check(x, "x", dims=2)
        n = expert_ids.numel()
        xs = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
        row_bytes = x.shape[1] * x.element_size()
        if n > 256 or row_bytes % 16 or x.data_ptr() % 16:
            plan = self.moe_plan(expert_ids, n_experts, tile_rows)
            self.gather_rows(x, plan.token_of, xs)
            return plan, xs
        plan, ptrs = self._plan_buffers(expert_ids, n_experts, tile_rows)
        self._run("moe", "flint_moe_dispatch", _ptr(expert_ids), c_int(n), c_int(n_experts), c_int(tile_rows), *ptrs,
                  c_int(plan.max_tiles), _ptr(x), _ptr(xs), c_int(row_bytes), c_int(plan.top))
        return plan, xs

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        _check(logits, "logits", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        self._run("sampling", "flint_argmax", _ptr(logits), _ptr(out), c_int(logits.shape[0]), c_int(logits.shape[1]))

    def sample(self, logits, params, context, work, out):
        """params [R, 8] float32: temperature, top_k, top_p, min_p, repeat_penalty, u, n_context, 0;
        context [R, C] int32 (recent tokens, -1 padded); work [R, V] float32 scratch."""
        _check(logits, "logits", torch.float32, 2)
        _check(params, "params", torch.float32, 2)
        _check(context, "context", torch.int32, 2)
        _check(work, "work", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        R, V = logits.shape
        if params.shape != (R, 8) or context.shape[0] != R or work.shape != (R, V) or out.numel() != R:
            raise KernelError("sample: shapes do not match")
        self._run("sampling", "flint_sample", _ptr(logits), _ptr(params), _ptr(context), c_int(context.shape[1]),
                  _ptr(work), _ptr(out), c_int(R), c_int(V))


_DEFAULT: dict = {}


def get_ops(device="cuda:0") -> CudaOps:
    key = str(torch.device(device))
    if key not in _DEFAULT:
        _DEFAULT[key] = CudaOps(device)
    return _DEFAULT[key]
