"""Thin, checked Python wrappers around the CUDA launchers of libcarbon_kernels.so.

Each wrapper takes torch tensors that live on the GPU, validates dtype and layout, and launches on
the current CUDA stream.  Nothing here computes on the CPU and nothing falls back to a library:
if the kernel library is missing or refuses a size, the call raises.
"""
from __future__ import annotations

import struct
from typing import Optional, Sequence

import torch

from .csrc.kernel_lib import KernelError, kernels

F32, BF16 = 0, 1
GEMM_STORE, GEMM_STORE_F32, GEMM_ACCUM_F32, GEMM_SWIGLU, GEMM_RELUGLU, GEMM_RELU2 = 0, 1, 2, 3, 4, 5      # 5: relu(v)^2, stored like 0
#: epilogues whose weight holds gate rows and up rows: act(gate) * up with act = SiLU or ReLU
GEMM_GATED = (GEMM_SWIGLU, GEMM_RELUGLU)
ROPE_PAIRINGS = {"half": 0, "interleaved": 1}


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dt} (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The current stream's handle (of the current device), the short way: this runs at every launch."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (replays of captured graphs included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


class KernelProfile:
    """Times every launch that goes through this module with CUDA events, one after each launch on the
    launching stream, while dependent launches are switched off so that kernels do not overlap: the time
    between two events is then the time of the kernel between them (plus its launch gap).  ``work`` that a
    caller notes before a launch (bytes it has to move, floating-point operations) is kept with it, so that
    :meth:`table` can set each kernel against the memory or arithmetic peak.  For measurement only: a
    profiled step is slower than a served one."""

    def __init__(self):
        self.records = []            # (kernel name, event after it, bytes, flops)
        self._work = (0, 0)
        self._start = None

    def __enter__(self):
        global _profile
        import torch
        self._pdl_before = _pdl_on
        set_dependent_launches(False)
        torch.cuda.synchronize()
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile
        import torch
        _profile = None
        torch.cuda.synchronize()
        set_dependent_launches(self._pdl_before)

    def note_work(self, nbytes: int, flops: int) -> None:
        self._work = (int(nbytes), int(flops))

    def mark(self) -> None:
        """The next launch's time counts from here (the step function marks the point where a step's host
        work and upload are done, so that they are not charged to the step's first kernel)."""
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.records.append((None, ev, 0, 0))

    def _launched(self, n: int) -> None:
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        name = kernels().ce_last_kernel().decode() or "?"
        self.records.append((name if n == 1 else f"{name} (+{n - 1})", ev, *self._work))
        self._work = (0, 0)

    def table(self, hbm_gbs: float, tflops: float, repeats: int = 1):
        """Rows (name, launches, microseconds per repeat, share, GB/s, TFLOP/s, fraction of the nearer
        peak) by kernel name, slowest first."""
        agg, prev, total = {}, self._start, 0.0
        for name, ev, nbytes, flops in self.records:
            us = prev.elapsed_time(ev) * 1e3
            prev = ev
            if name is None:             # a mark: what came before it is nobody's
                continue
            a = agg.setdefault(name, [0, 0.0, 0, 0])
            a[0] += 1; a[1] += us; a[2] += nbytes; a[3] += flops
            total += us
        rows = []
        for name, (n, us, nbytes, flops) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            gbs = nbytes / us / 1e3 if us > 0 else 0.0
            tf = flops / us / 1e6 if us > 0 else 0.0
            frac = max(gbs / hbm_gbs, tf / tflops) if (nbytes or flops) else None
            rows.append({"kernel": name, "launches": n // repeats, "us": round(us / repeats, 1), "share": round(us / total, 4),
                         "gb_s": round(gbs, 1), "tflop_s": round(tf, 1), "frac_of_peak": None if frac is None else round(frac, 3)})
        return rows, total / repeats


_profile: Optional[KernelProfile] = None


def profiling() -> Optional[KernelProfile]:
    return _profile


def _ok(code: int, n: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(kernels().ce_last_error().decode())
    _launches += n
    if _profile is not None:
        _profile._launched(n)


_pdl_on = True


def set_dependent_launches(on: bool) -> None:
    """Whether kernels launched from now on may start while the kernel before them still runs (programmatic
    dependent launch).  The step function turns it off for steps of many tokens, see ``ModelRunner.step``."""
    global _pdl_on
    if bool(on) != _pdl_on:
        kernels().ce_set_pdl(1 if on else 0)
        _pdl_on = bool(on)


def kernel_counts() -> dict:
    """Launches so far by kernel name (a launch captured in a CUDA graph counts once, at capture): shows
    WHICH kernel took each shape."""
    import ctypes
    k = kernels()
    need = k.ce_kernel_counts(None, 0)
    buf = ctypes.create_string_buffer(need + 64)
    k.ce_kernel_counts(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, _, n = line.rpartition("=")
        out[name] = int(n)
    return out


def reset_kernel_counts() -> None:
    kernels().ce_kernel_counts_reset()


def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """x[t, :] = table[tokens[t], :] * scale as float32."""
    _need(table, "table"); _need(tokens, "tokens", torch.int32); _need(x, "x", torch.float32)
    T, H = x.shape
    _ok(kernels().ce_embed(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(x), T, H, table.shape[0],
                           _ptr(status), float(scale), _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32, out float32 or bfloat16."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    R, H = out.shape
    if x.shape[1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: widths differ: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _ok(kernels().ce_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), R, H, float(eps),
                             _stream()))


def qk_rope_kvwrite(qkv, k_pool, v_pool, q_weight, k_weight, cos, sin, positions, seq_of_token, seq_slot,
                    block_table, status, nh: int, nkv: int, d: int, rotary_dim: int, page_size: int,
                    eps: float, write_kv: bool = True, pairing: str = "half") -> None:
    """Per-head q/k RMSNorm, rotation, and the write of K and V into the pages.  ``pairing``: which elements
    of a head turn together, "half" (i with i + rotary_dim/2) or "interleaved" (2i with 2i + 1)."""
    _need(qkv, "qkv")
    if pairing not in ROPE_PAIRINGS:
        raise KernelError(f"qk_rope_kvwrite: unknown pairing '{pairing}' (half, interleaved)")
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qk_rope_kvwrite: qkv width {qkv.shape[1]} != (nh + 2 nkv) d = {(nh + 2 * nkv) * d}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight), ("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32)
    max_pos = cos.shape[0] if cos is not None else 0
    if cos is not None and cos.shape[1] != rotary_dim // 2:
        raise KernelError("qk_rope_kvwrite: rotary table width is not rotary_dim / 2")
    if write_kv:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype)
        if tuple(k_pool.shape[1:]) != (nkv, page_size, d):
            raise KernelError(f"qk_rope_kvwrite: pool shape {tuple(k_pool.shape)} is not [pages, {nkv}, {page_size}, {d}]")
    num_pages = k_pool.shape[0] if k_pool is not None else 0
    max_pages = block_table.shape[1] if block_table is not None else 0
    _ok(kernels().ce_qk_rope_kvwrite(
        _ptr(qkv), _ptr(k_pool), _ptr(v_pool), dtype_code(qkv.dtype), _ptr(q_weight), _ptr(k_weight), _ptr(cos),
        _ptr(sin), _ptr(positions), _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status),
        T, nh, nkv, d, rotary_dim, page_size, max_pages, num_pages, max_pos, 1 if write_kv else 0, float(eps),
        ROPE_PAIRINGS[pairing], _stream()))


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x, "x", torch.float32); _need(delta, "delta")
    if x.numel() != delta.numel():
        raise KernelError("add_residual: sizes differ")
    _ok(kernels().ce_add_residual(_ptr(x), _ptr(delta), dtype_code(delta.dtype), x.numel(), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError("swiglu: gate_up must be [T, 2I]")
    _ok(kernels().ce_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I, _stream()))


def reluglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = relu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError("reluglu: gate_up must be [T, 2I]")
    _ok(kernels().ce_reluglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I, _stream()))


def relu2(inp: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = relu(inp[t, i])^2; inp contiguous [T, I], out rows of stride out.stride(0)."""
    _need(inp, "inp")
    if out.dtype != inp.dtype or out.shape != inp.shape or out.stride(-1) != 1 or not out.is_cuda:
        raise KernelError("relu2: shapes or dtypes do not fit")
    _ok(kernels().ce_relu2(_ptr(inp), _ptr(out), dtype_code(out.dtype), inp.shape[0], inp.shape[1], out.stride(0), _stream()))


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, eps: float,
              rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x - mean) / sqrt(var + eps) * weight + bias of row rows[r] (or r); x float32."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(bias, "bias", torch.float32); _need(out, "out")
    R, H = out.shape
    if x.shape[1] != H or weight.numel() != H or bias.numel() != H:
        raise KernelError(f"layernorm: widths differ: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _ok(kernels().ce_layernorm(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), dtype_code(out.dtype), _ptr(rows), R, H, float(eps),
                               _stream()))


def rmsnorm_add(y: torch.Tensor, weight: torch.Tensor, x: torch.Tensor, eps: float, rounded: Optional[torch.Tensor] = None) -> None:
    """x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight; all float32.  ``rounded`` (bfloat16, the shape of x, contiguous)
    receives the new x rounded: the input of a sublayer that reads the residual itself."""
    _need(y, "y", torch.float32); _need(weight, "weight", torch.float32); _need(x, "x", torch.float32)
    if y.shape != x.shape or weight.numel() != x.shape[1]:
        raise KernelError("rmsnorm_add: sizes differ")
    if rounded is not None:
        _need(rounded, "rounded", torch.bfloat16)
        if rounded.shape != x.shape:
            raise KernelError("rmsnorm_add: the rounded copy must have the shape of x")
    _ok(kernels().ce_rmsnorm_add(_ptr(y), _ptr(weight), _ptr(x), _ptr(rounded), x.shape[0], x.shape[1], float(eps), _stream()))


def tanh_cap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _need(x, "x", torch.float32)
    _ok(kernels().ce_tanh_cap(_ptr(x), x.numel(), float(cap), _stream()))


def copy_cols(src: torch.Tensor, off: int, width: int, out: torch.Tensor) -> None:
    """out[t, l] = src[t, off + l] for l < width; src float32 (row stride src.stride(0)), out float32 or bfloat16."""
    _need(out, "out")
    if src.dtype != torch.float32 or src.stride(-1) != 1 or not src.is_cuda:
        raise KernelError("copy_cols: src must be float32 rows on the GPU")
    if out.shape != (src.shape[0], width) or off + width > src.shape[1]:
        raise KernelError("copy_cols: sizes do not fit")
    _ok(kernels().ce_copy_cols(_ptr(src), _ptr(out), dtype_code(out.dtype), src.shape[0], src.stride(0), int(off), int(width),
                               _stream()))


def side_gate(z: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, off: int, status) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], off + j]; z float32 [T, D], out in the table's dtype."""
    _need(z, "z", torch.float32); _need(table, "table"); _need(tokens, "tokens", torch.int32); _need(out, "out", table.dtype)
    T, D = z.shape
    if out.shape != z.shape:
        raise KernelError("side_gate: sizes differ")
    _ok(kernels().ce_side_gate(_ptr(z), _ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), T, D, table.shape[1],
                               int(off), table.shape[0], _ptr(status), _stream()))


def value_mix(rows: torch.Tensor, off: int, n: int, first: torch.Tensor, first_off: int, lam: float) -> None:
    """rows[:, off:off+n] <- (1 - lam) rows[:, off:off+n] + lam first[:, first_off:first_off+n], in place."""
    if rows.dtype != first.dtype or rows.stride(-1) != 1 or first.stride(-1) != 1 or rows.shape[0] != first.shape[0]:
        raise KernelError("value_mix: the two row sets must agree in dtype and token count")
    if off + n > rows.shape[1] or first_off + n > first.shape[1]:
        raise KernelError("value_mix: columns outside a row")
    _ok(kernels().ce_value_mix(_ptr(rows), dtype_code(rows.dtype), rows.stride(0), int(off), int(n), _ptr(first), first.stride(0),
                               int(first_off), float(lam), rows.shape[0], _stream()))


def latent_prepare(proj, wq, wkv, cq, k_pool, cos, sin, positions, seq_of_token, seq_slot, block_table, status, off_q: int,
                   qr: int, off_kv: int, r: int, dr: int, rd: int, page_size: int, eps: float, write_kv: bool = True) -> None:
    """Latent attention's operands from one float32 product row: cq = rms_norm(query latent) * wq; the token's
    cache row [rms_norm(latent) * wkv | rotated key part] into ``k_pool`` [pages, 1, page, r + dr]."""
    _need(proj, "proj", torch.float32)
    if qr > 0:
        _need(wq, "wq", torch.float32); _need(cq, "cq")
    if (qr > 0 and (cq.shape != (proj.shape[0], qr) or wq.numel() != qr)) or (write_kv and (wkv is None or wkv.numel() != r)):
        raise KernelError("latent_prepare: sizes do not fit")
    if write_kv:
        _need(wkv, "wkv", torch.float32)
        _need(k_pool, "k_pool", cq.dtype if qr > 0 else None)
        if tuple(k_pool.shape[1:]) != (1, page_size, r + dr):
            raise KernelError(f"latent_prepare: pool {tuple(k_pool.shape)} is not [pages, 1, {page_size}, {r + dr}]")
    if rd > 0 and (cos is None or cos.shape[1] != rd // 2):
        raise KernelError("latent_prepare: rotary table width is not rd / 2")
    _ok(kernels().ce_latent_prepare(
        _ptr(proj), _ptr(wq), _ptr(wkv), _ptr(cq), _ptr(k_pool), dtype_code(cq.dtype if qr > 0 else k_pool.dtype), _ptr(cos), _ptr(sin), _ptr(positions),
        _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status), proj.shape[0], proj.stride(0), int(off_q), int(qr),
        int(off_kv), int(r), int(dr), int(rd), int(page_size), block_table.shape[1] if block_table is not None else 0,
        k_pool.shape[0] if k_pool is not None else 0, cos.shape[0] if cos is not None else 0, 1 if write_kv else 0, float(eps),
        _stream()))


def rope_part(src, src_head: int, src_off: int, dst, dst_head: int, dst_off: int, cos, sin, positions, status, heads: int,
              dr: int, rd: int) -> None:
    """dst[t, h*dst_head + dst_off + i] = src[t, h*src_head + src_off + i] for i < dr, its first rd elements rotated in half pairs."""
    if src.dtype != dst.dtype or src.stride(-1) != 1 or dst.stride(-1) != 1:
        raise KernelError("rope_part: rows of one dtype are needed")
    _ok(kernels().ce_rope_part(_ptr(src), src.stride(0), int(src_head), int(src_off), _ptr(dst), dst.stride(0), int(dst_head),
                               int(dst_off), dtype_code(src.dtype), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(status),
                               src.shape[0], int(heads), int(dr), int(rd), cos.shape[0] if cos is not None else 0, _stream()))


def head_matmul(inp, in_head: int, w, out, out_head: int, heads: int, n: int, k: int, gate=None, gate_per_head: bool = False) -> None:
    """out[t, h*out_head + j] = sum_i inp[t, h*in_head + i] * w[h, j, i] (j < n, i < k), optionally times
    sigmoid(gate[t, h*n + j]) or, with ``gate_per_head``, sigmoid(gate[t, h]) (float32 logits); w [heads, n, k]
    contiguous, operands and output in one dtype."""
    _need(w, "w", inp.dtype)
    if tuple(w.shape) != (heads, n, k) or out.dtype != inp.dtype or inp.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("head_matmul: shapes or dtypes do not fit")
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(-1) != 1):
        raise KernelError("head_matmul: the gate logits must be float32 rows")
    prof = profiling()
    if prof is not None:
        M = inp.shape[0]
        prof.note_work((M * heads * (n + k) + heads * n * k) * inp.element_size(), 2 * M * heads * n * k)
    _ok(kernels().ce_head_matmul(_ptr(inp), inp.stride(0), int(in_head), _ptr(w), _ptr(out), out.stride(0), int(out_head),
                                 _ptr(gate), gate.stride(0) if gate is not None else 0, 1 if gate_per_head else 0,
                                 dtype_code(inp.dtype), inp.shape[0],
                                 int(heads), int(n), int(k), _stream()))


def masked_attention(q, q_head: int, k_pool, v_pool, ldk: int, ldv: int, gate, out, positions, seq_of_token, seq_slot,
                     block_table, status, nh: int, nkv: int, d: int, dv: int, page_size: int, window: int, keep_first: int,
                     scale: float, softcap: float, sinks=None, out_scale: float = 1.0) -> None:
    """Softmax attention in float32 arithmetic with separate key and value head sizes, a tanh cap on the scores
    (0: none), a window (0: none) that keeps the first ``keep_first`` keys visible, and an optional sigmoid gate per
    output element.  ``v_pool`` may be the key pool itself (``ldv`` = ``ldk``): the values are then the leading
    ``dv`` elements of every key row.  ``sinks`` (float32 [nh]): exp(sinks[h]) is one more term of head h's denominator."""
    _need(k_pool, "k_pool"); _need(out, "out", k_pool.dtype)
    _check_sinks(sinks, nh)
    if q.dtype != k_pool.dtype or v_pool.dtype != k_pool.dtype:
        raise KernelError("masked_attention: q and the cache differ in dtype")
    _ok(kernels().ce_masked_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(gate), _ptr(out), dtype_code(out.dtype), _ptr(positions), _ptr(seq_of_token),
        _ptr(seq_slot), _ptr(block_table), _ptr(status), out.shape[0], nh, nkv, d, dv, q.stride(0), int(q_head), int(ldk), int(ldv),
        gate.stride(0) if gate is not None else 0, page_size, block_table.shape[1], k_pool.shape[0], int(window), int(keep_first),
        float(scale), float(softcap), _ptr(sinks), float(out_scale), _stream()))


def _check_sinks(sinks, nh: int) -> None:
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != nh or not sinks.is_contiguous() or not sinks.is_cuda):
        raise KernelError(f"attention sinks must be {nh} float32 numbers on the GPU")


def masked_attention_mma_supported(d: int, dv: int, q_stride: int, q_head: int, ldk: int, ldv: int, alias: bool) -> bool:
    return bool(kernels().ce_masked_attention_mma_supported(d, dv, q_stride, q_head, ldk, ldv, 1 if alias else 0))


def masked_attention_mma(q, q_head: int, k_pool, v_pool, ldk: int, ldv: int, gate, out, positions, seq_slot, q_start, block_table,
                         tiles, n_tiles: int, status, nh: int, nkv: int, d: int, dv: int, page_size: int, window: int,
                         keep_first: int, scale: float, softcap: float, sinks=None, out_scale: float = 1.0) -> None:
    """:func:`masked_attention` on the tensor cores (bfloat16) for tiles of 64 query tokens: ``tiles`` holds (sequence, first
    token within the sequence's tokens of the step) pairs.  ``gate`` holds bfloat16 logits."""
    _need(k_pool, "k_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    if q.dtype != torch.bfloat16 or v_pool.dtype != torch.bfloat16 or (gate is not None and gate.dtype != torch.bfloat16):
        raise KernelError("masked_attention_mma: bfloat16 only")
    _check_sinks(sinks, nh)
    _ok(kernels().ce_masked_attention_mma(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(gate), _ptr(out), _ptr(positions), _ptr(seq_slot), _ptr(q_start), _ptr(block_table),
        _ptr(tiles), _ptr(status), int(n_tiles), out.shape[0], nh, nkv, d, dv, q.stride(0), int(q_head), int(ldk), int(ldv),
        gate.stride(0) if gate is not None else 0, page_size, block_table.shape[1], k_pool.shape[0], int(window), int(keep_first),
        float(scale), float(softcap), _ptr(sinks), float(out_scale), _stream()))


def norm_rope_kvwrite(proj, q_out, k_pool, v_pool, wq, wk, head_scale, cos, sin, positions, seq_of_token, seq_slot, block_table,
                      status, off_q: int, off_k: int, off_v: int, nh: int, nkv: int, d: int, dv: int, rotary_dim: int,
                      page_size: int, eps: float, write_kv: bool = True) -> None:
    """Operands of attention with a norm per head, from float32 rows ``proj``: query heads (from ``off_q``) and key heads
    (from ``off_k``) divided by their root mean square times ``wq`` / ``wk`` (None: no norm), rotated over their first
    ``rotary_dim`` elements (element i with i + rotary_dim/2), queries times ``head_scale[h]`` (None: no factor) into
    ``q_out`` [T, nh * d], keys and the values (``nkv`` heads of ``dv`` from ``off_v``; ``off_v`` = ``off_k``: the keys as
    projected) into the pages."""
    _need(q_out, "q_out")
    if proj.dtype != torch.float32 or proj.stride(-1) != 1:
        raise KernelError("norm_rope_kvwrite: proj must be float32 rows")
    for name, t in (("wq", wq), ("wk", wk), ("head_scale", head_scale), ("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32)
    T = q_out.shape[0]
    if q_out.shape[1] != nh * d or (wq is not None and wq.numel() != d) or (wk is not None and wk.numel() != d) or \
            (head_scale is not None and head_scale.numel() != nh) or proj.shape[1] < max(off_q + nh * d, off_k + nkv * d, off_v + nkv * dv):
        raise KernelError("norm_rope_kvwrite: sizes do not fit")
    if cos is not None and cos.shape[1] != rotary_dim // 2:
        raise KernelError("norm_rope_kvwrite: rotary table width is not rotary_dim / 2")
    if write_kv:
        _need(k_pool, "k_pool", q_out.dtype); _need(v_pool, "v_pool", q_out.dtype)
        if tuple(k_pool.shape[1:]) != (nkv, page_size, d) or tuple(v_pool.shape[1:]) != (nkv, page_size, dv):
            raise KernelError(f"norm_rope_kvwrite: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit "
                              f"{nkv} x {d} keys and {nkv} x {dv} values in pages of {page_size}")
    _ok(kernels().ce_norm_rope_kvwrite(
        _ptr(proj), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), dtype_code(q_out.dtype), _ptr(wq), _ptr(wk), _ptr(head_scale),
        _ptr(cos), _ptr(sin), _ptr(positions), _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status), T,
        proj.stride(0), int(off_q), int(off_k), int(off_v), nh, nkv, d, dv, rotary_dim if cos is not None else 0, page_size,
        block_table.shape[1] if block_table is not None else 0, k_pool.shape[0] if k_pool is not None else 0,
        cos.shape[0] if cos is not None else 0, 1 if write_kv else 0, float(eps), _stream()))


def gated_delta_prep_width(heads: int, key_heads: int, d: int, dv: int) -> int:
    return kernels().ce_gated_delta_prep_width(heads, key_heads, d, dv)


DECAY_PER_CHANNEL, DECAY_PER_HEAD, DECAY_CONSTANT = 0, 1, 2
GATE_SIGMOID, GATE_SILU = 0, 1


def gated_delta(proj, dec, gz, taps, a_log, dt_bias, norm_w, prep, raw, state, kept, out, seq_of_token, seq_slot, q_start,
                n_seqs: int, off_conv: int, off_b: int, heads: int, key_heads: int, d: int, dv: int, n_taps: int, eps: float,
                decay: int = DECAY_PER_CHANNEL, gate: int = GATE_SIGMOID, delta: bool = True, out_scale: float = 1.0,
                rotation=None) -> None:
    """The recurrent mixers with a matrix state per head over each sequence's tokens of the step, from and to ``state``
    [slots, heads, d, dv] (float32).  ``proj`` float32 [T, ld] holds q | k | v from ``off_conv`` and the beta logits at
    ``off_b``; ``gz`` the gate logits [T, heads * dv] (rows of any stride).

    ``delta``: the gated delta rule (True) or the plain decaying sum of outer products, which writes v itself (False).
    ``decay``: per head and key channel from logits ``dec`` [T, heads * d] with ``dt_bias`` [heads * d]; per head from
    logits ``dec`` [T, heads] with ``dt_bias`` [heads]; or constant, ``a_log`` then holding the heads' decays themselves.
    ``rotation`` None: q, k, v pass the short convolution (``taps`` [C, n_taps], the kept rows ``kept`` [slots, taps - 1, C])
    and SiLU, and q and k become unit vectors; ``rotation`` = (cos, sin, rotary_dim, positions, status): no convolution, q and
    k are rotated by the position and k is multiplied by d^-1/2 (with constant decays).  ``gate``: sigmoid or SiLU of the
    gate logits; ``norm_w`` None: no weight after the root mean square; ``out_scale`` multiplies what is stored.
    Four launches: prepare, keep, walk, finish."""
    _need(state, "state", torch.float32); _need(out, "out")
    for name, t in (("taps", taps), ("a_log", a_log), ("dt_bias", dt_bias), ("norm_w", norm_w), ("prep", prep), ("raw", raw)):
        if t is not None:
            _need(t, name, torch.float32)
    for name, t in (("proj", proj), ("dec", dec), ("gz", gz)):
        if t is not None and (t.dtype != torch.float32 or t.stride(-1) != 1 or not t.is_cuda):
            raise KernelError(f"gated_delta: {name} must be float32 rows on the GPU")
    T, C = out.shape[0], 2 * key_heads * d + heads * dv
    P = gated_delta_prep_width(heads, key_heads, d, dv)
    n_dec = {DECAY_PER_CHANNEL: heads * d, DECAY_PER_HEAD: heads}.get(decay)
    if tuple(state.shape[1:]) != (heads, d, dv) or out.shape[1] != heads * dv or tuple(gz.shape) != (T, heads * dv) or \
            prep.numel() < T * P or raw.numel() < T * heads * dv or a_log.numel() != heads or \
            (norm_w is not None and norm_w.numel() != dv):
        raise KernelError("gated_delta: sizes do not fit")
    if n_dec is not None and (dec is None or tuple(dec.shape) != (T, n_dec) or dt_bias is None or dt_bias.numel() != n_dec):
        raise KernelError("gated_delta: the decay's logits or bias do not fit")
    cos = sin = positions = status = None
    rd = max_pos = 0
    if rotation is None:
        if tuple(taps.shape) != (C, n_taps) or (n_taps > 1 and tuple(kept.shape[1:]) != (n_taps - 1, C)):
            raise KernelError("gated_delta: the convolution's sizes do not fit")
    else:
        cos, sin, rd, positions, status = rotation
        if n_taps != 1 or decay != DECAY_CONSTANT:
            raise KernelError("gated_delta: rotated operands come without a convolution and with constant decays")
        if cos is not None:
            _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32)
            if cos.shape[1] != rd // 2:
                raise KernelError("gated_delta: rotary table width is not rotary_dim / 2")
            max_pos = cos.shape[0]
        else:
            rd = 0
    prof, work = profiling(), None
    if prof is not None:
        work, prof._work = prof._work, (0, 0)            # the caller's figures belong to the walk
    for stage in (1, 2, 3, 4):
        if stage == 2 and n_taps == 1:
            continue
        if stage == 3 and work is not None:
            prof.note_work(*work)
        _ok(kernels().ce_gated_delta(_ptr(proj), _ptr(dec), _ptr(gz), _ptr(taps), _ptr(a_log), _ptr(dt_bias), _ptr(norm_w),
                                     _ptr(prep), _ptr(raw), _ptr(state), _ptr(kept), _ptr(out), dtype_code(out.dtype),
                                     _ptr(seq_of_token), _ptr(seq_slot), _ptr(q_start), T, n_seqs, proj.stride(0), int(off_conv),
                                     int(off_b), heads, key_heads, d, dv, n_taps, float(eps),
                                     dec.stride(0) if dec is not None else 0, gz.stride(0), int(decay), 0 if rotation is None else 1,
                                     0 if delta else 1, int(gate), float(out_scale), _ptr(cos), _ptr(sin), _ptr(positions),
                                     _ptr(status), int(rd), int(max_pos), stage, _stream()))


def attention_generic(q, q_stride: int, k_pool, v_pool, out, positions, seq_of_token, seq_slot, block_table,
                      status, nh: int, nkv: int, d: int, page_size: int, window: int, scale: float,
                      T: Optional[int] = None) -> None:
    _need(k_pool, "k_pool"); _need(v_pool, "v_pool", k_pool.dtype); _need(out, "out", k_pool.dtype)
    if q.dtype != k_pool.dtype:
        raise KernelError("attention: q and the cache differ in dtype")
    T = out.shape[0] if T is None else T
    _ok(kernels().ce_attention_generic(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), dtype_code(out.dtype), _ptr(positions), _ptr(seq_of_token),
        _ptr(seq_slot), _ptr(block_table), _ptr(status), T, nh, nkv, d, q_stride, page_size, block_table.shape[1],
        k_pool.shape[0], int(window), float(scale), _stream()))


def gemm_plain(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, mode: int) -> None:
    """c = a @ w.T with float32 FMA arithmetic; see csrc/kernels/gemm_plain.cu for the epilogues."""
    _need(w, "w", a.dtype); _need(c, "c")
    if a.stride(-1) != 1 or c.stride(-1) != 1:
        raise KernelError("gemm_plain: rows must be contiguous")
    M, K = a.shape
    N = c.shape[1]
    rows = 2 * N if mode in GEMM_GATED else N
    if w.shape != (rows, K) or c.shape[0] != M:
        raise KernelError(f"gemm_plain: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)} do not fit")
    want = torch.float32 if mode in (GEMM_STORE_F32, GEMM_ACCUM_F32) else a.dtype
    if c.dtype != want:
        raise KernelError(f"gemm_plain: output must be {want}")
    _ok(kernels().ce_gemm_plain(_ptr(a), _ptr(w), _ptr(c), dtype_code(a.dtype), M, N, K, a.stride(0), c.stride(0),
                                mode, _stream()))


def streams_norm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, groups: int = 1,
                 coef: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = RMS norm in ``groups`` equal parts of sum_s coef[s] x[row, s, :], times weight.  x float32
    [T, W] or [T, S, W]; coef None: the plain sum of the streams."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    R, W = out.shape
    S = x.shape[1] if x.dim() == 3 else 1
    if x.shape[-1] != W or weight.numel() != W:
        raise KernelError(f"streams_norm: widths differ: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if coef is not None:
        _need(coef, "coef", torch.float32)
        if coef.numel() != S:
            raise KernelError(f"streams_norm: {coef.numel()} coefficients for {S} streams")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _ok(kernels().ce_streams_norm(_ptr(x), _ptr(coef), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), R, S, W,
                                  int(groups), float(eps), _stream()))


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, out: torch.Tensor, positions, seq_of_token,
                seq_slot, q_start, save: bool = True) -> None:
    """out[t] = h[t] + (previous row - h[t]) * mu; the previous row of a portion's first token is state[slot]
    (zeros at position 0).  h and state float32.  ``save``: state[slot] then becomes the portion's last row."""
    _need(h, "h", torch.float32); _need(mu, "mu", torch.float32); _need(state, "state", torch.float32); _need(out, "out")
    T, W = h.shape
    if out.shape != h.shape or mu.numel() != W or state.shape[-1] != W:
        raise KernelError("token_shift: sizes differ")
    _ok(kernels().ce_token_shift(_ptr(h), _ptr(mu), _ptr(state), _ptr(out), dtype_code(out.dtype), _ptr(positions),
                                 _ptr(seq_of_token), _ptr(seq_slot), _ptr(q_start), T, W, 1 if save else 0, _stream()))


def save_last_rows(h: torch.Tensor, state: torch.Tensor, seq_slot: torch.Tensor, q_start: torch.Tensor) -> None:
    """state[slot of sequence b] = h[last token of b] for every sequence of the step."""
    _need(h, "h", torch.float32); _need(state, "state", torch.float32)
    if state.shape[-1] != h.shape[1]:
        raise KernelError("save_last_rows: widths differ")
    _ok(kernels().ce_save_last_rows(_ptr(h), _ptr(state), _ptr(seq_slot), _ptr(q_start), seq_slot.numel(), h.shape[1],
                                    _stream()))


def streams_write(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, c_out: torch.Tensor,
                  bias: Optional[torch.Tensor] = None) -> None:
    """x[t, to] <- sum_from mix[from, to] x[t, from] + c_out[to] (y[t] + bias), in place; x [T, S, W] float32."""
    _need(x, "x", torch.float32); _need(y, "y", torch.float32); _need(mix, "mix", torch.float32)
    _need(c_out, "c_out", torch.float32)
    T, S, W = x.shape
    if y.shape != (T, W) or mix.shape != (S, S) or c_out.numel() != S:
        raise KernelError(f"streams_write: x {tuple(x.shape)}, y {tuple(y.shape)}, mix {tuple(mix.shape)} do not fit")
    _ok(kernels().ce_streams_write(_ptr(x), _ptr(y), _ptr(mix), _ptr(c_out), _ptr(bias), T, S, W, _stream()))


def streams_broadcast(x0: torch.Tensor, x: torch.Tensor) -> None:
    """x[t, s] = x0[t] for every stream s."""
    _need(x0, "x0", torch.float32); _need(x, "x", torch.float32)
    T, S, W = x.shape
    if x0.shape != (T, W):
        raise KernelError("streams_broadcast: sizes differ")
    _ok(kernels().ce_streams_broadcast(_ptr(x0), _ptr(x), T, S, W, _stream()))


def add_bias(out: torch.Tensor, bias: torch.Tensor, n: Optional[int] = None) -> None:
    """out[:, :n] += bias (float32), out float32 or bfloat16."""
    _need(out, "out"); _need(bias, "bias", torch.float32)
    n = bias.numel() if n is None else n
    if n > out.shape[1] or n > bias.numel():
        raise KernelError("add_bias: more columns than the output or the bias has")
    _ok(kernels().ce_add_bias(_ptr(out), dtype_code(out.dtype), _ptr(bias), out.shape[0], n, out.stride(0), _stream()))


def bias_rope_kvwrite(qkv, k_pool, v_pool, bias, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
                      nq: int, nk: int, nv: int, d: int, dv: int, rotary_dim: int, page_size: int,
                      write_kv: bool = True) -> None:
    """Rows [nq heads of d | nk heads of d | nv heads of dv | ...]: bias added, q and k rotated over their first
    ``rotary_dim`` elements (element i with i + rotary_dim/2), q in place, k and v into the pages."""
    _need(qkv, "qkv")
    for name, t in (("bias", bias), ("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32)
    if bias is not None and bias.numel() < (nq + nk) * d + nv * dv:
        raise KernelError("bias_rope_kvwrite: the bias is shorter than q|k|v")
    if cos is not None and cos.shape[1] != rotary_dim // 2:
        raise KernelError("bias_rope_kvwrite: rotary table width is not rotary_dim / 2")
    if write_kv:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype)
        if tuple(k_pool.shape[1:]) != (nk, page_size, d) or tuple(v_pool.shape[1:]) != (nv, page_size, dv):
            raise KernelError(f"bias_rope_kvwrite: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit "
                              f"{nk} x {d} keys and {nv} x {dv} values in pages of {page_size}")
    _ok(kernels().ce_bias_rope_kvwrite(
        _ptr(qkv), _ptr(k_pool), _ptr(v_pool), dtype_code(qkv.dtype), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(positions),
        _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status), qkv.shape[0], qkv.stride(0), nq, nk, nv, d, dv,
        rotary_dim if cos is not None else 0, page_size, block_table.shape[1] if block_table is not None else 0,
        k_pool.shape[0] if k_pool is not None else 0, cos.shape[0] if cos is not None else 0, 1 if write_kv else 0, _stream()))


def diff_attention(q, q_stride: int, k_pool, v_pool, gate, gate_stride: int, out, positions, seq_of_token, seq_slot,
                   block_table, status, nh: int, nkv: int, d: int, dv: int, page_size: int, window: int, chunk: int,
                   scale: float, lam: float, eps: float, out_scale: float, n_tokens: Optional[int] = None) -> None:
    """Differential attention in float32 arithmetic (``n_tokens``: only the first so many tokens of the step): two softmax maps per head over the same values,
    o = a1 - lam a2, unit RMS per head times ``out_scale``, times sigmoid(gate logit)."""
    _need(k_pool, "k_pool"); _need(v_pool, "v_pool", k_pool.dtype); _need(out, "out", k_pool.dtype)
    if q.dtype != k_pool.dtype:
        raise KernelError("diff_attention: q and the cache differ in dtype")
    if k_pool.shape[1] != 2 * nkv or k_pool.shape[3] != d or v_pool.shape[1] != nkv or v_pool.shape[3] != dv:
        raise KernelError(f"diff_attention: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit {nkv} key heads")
    _ok(kernels().ce_diff_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(gate), _ptr(out), dtype_code(out.dtype), _ptr(positions),
        _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status), out.shape[0], nh, nkv, d, dv, q_stride,
        gate_stride, page_size, block_table.shape[1], k_pool.shape[0], int(window), int(chunk), float(scale), float(lam),
        float(eps), float(out_scale), _stream()))


def diff_attention_mma_supported(d: int, dv: int, q_stride: int) -> bool:
    return bool(kernels().ce_diff_attention_mma_supported(d, dv, q_stride))


def diff_attention_mma(q, q_stride: int, k_pool, v_pool, gate, gate_stride: int, out, positions, seq_slot, q_start,
                       block_table, tiles, n_tiles: int, status, nh: int, nkv: int, d: int, dv: int, page_size: int,
                       window: int, chunk: int, scale: float, lam: float, eps: float, out_scale: float) -> None:
    """Differential attention on the tensor cores (bfloat16) for tiles of 64 query tokens: ``tiles`` holds
    (sequence, first token within the sequence's tokens of the step) pairs."""
    _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    if q.dtype != torch.bfloat16:
        raise KernelError("diff_attention_mma: bfloat16 only")
    if k_pool.shape[1] != 2 * nkv or k_pool.shape[3] != d or v_pool.shape[1] != nkv or v_pool.shape[3] != dv:
        raise KernelError(f"diff_attention_mma: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit {nkv} key heads")
    _ok(kernels().ce_diff_attention_mma(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(gate), _ptr(out), _ptr(positions), _ptr(seq_slot), _ptr(q_start),
        _ptr(block_table), _ptr(tiles), _ptr(status), int(n_tiles), nh, nkv, d, dv, q_stride, gate_stride, page_size,
        block_table.shape[1], k_pool.shape[0], int(window), int(chunk), float(scale), float(lam), float(eps),
        float(out_scale), _stream()))


def tanh_cols(proj: torch.Tensor, off: int, width: int, out: torch.Tensor) -> None:
    """out[t, l] = tanh(proj[t, off + l]) for l < width; proj float32, out float32 or bfloat16 [T, width]."""
    _need(proj, "proj", torch.float32); _need(out, "out")
    if out.shape != (proj.shape[0], width) or off + width > proj.shape[1]:
        raise KernelError("tanh_cols: sizes do not fit")
    _ok(kernels().ce_tanh_cols(_ptr(proj), _ptr(out), dtype_code(out.dtype), proj.shape[0], proj.stride(0), int(off),
                               int(width), _stream()))


def general_delta(proj, zz, w0, a_bias, norm_w, prep, raw, state, out, seq_slot, q_start, n_seqs: int,
                  offsets: Sequence[int], heads: int, d: int, eps: float) -> None:
    """The generalized delta rule over each sequence's tokens of the step, from and to ``state``
    [slots, heads, d, d] (float32).  ``proj`` float32 [T, ld] holds, at ``offsets`` (r, k, v, a, g), the
    projections of every token, ``zz`` [T, heads * d] the decay logits; ``prep`` [T, 3 * heads * d] and ``raw``
    [T, heads * d] are float32 work space; ``out`` [T, heads * d] receives the normed, gated outputs.  Three
    launches: prepare, walk, finish."""
    _need(proj, "proj", torch.float32); _need(state, "state", torch.float32); _need(out, "out")
    for name, t in (("zz", zz), ("w0", w0), ("a_bias", a_bias), ("norm_w", norm_w), ("prep", prep), ("raw", raw)):
        _need(t, name, torch.float32)
    T, n = out.shape[0], heads * d
    if tuple(state.shape[1:]) != (heads, d, d) or out.shape[1] != n or zz.shape != (T, n) or prep.numel() < 3 * T * n \
            or raw.numel() < T * n:
        raise KernelError("general_delta: sizes do not fit")
    off_r, off_k, off_v, off_a, off_g = (int(o) for o in offsets)
    prof, work = profiling(), None
    if prof is not None:
        work, prof._work = prof._work, (0, 0)            # the caller's figures belong to the walk
    for stage in (1, 2, 3):
        if stage == 2 and work is not None:
            prof.note_work(*work)
        _ok(kernels().ce_general_delta(_ptr(proj), _ptr(zz), _ptr(w0), _ptr(a_bias), _ptr(norm_w), _ptr(prep), _ptr(raw),
                                       _ptr(state), _ptr(out), dtype_code(out.dtype), _ptr(seq_slot), _ptr(q_start), T, n_seqs,
                                       proj.stride(0), off_r, off_k, off_v, off_a, off_g, heads, d, float(eps), stage, _stream()))


MOE_ACTIVATIONS = {"none": 0, "relu2": 1}


def moe_route(z: torch.Tensor, experts: int, top: int, groups: int, keep: int, scale: float, ids: torch.Tensor,
              weights: torch.Tensor, sgate: Optional[torch.Tensor] = None) -> None:
    """Router logits z [T, >= experts (+1)] float32 -> the ``top`` experts of every token (``ids`` int32 [T, top], best
    first) and their weights (float32 [T, top]): softmax over the experts, experts in ``groups`` equal groups of neighbours
    of which the ``keep`` with the largest member stay eligible, weights = chosen scores / their sum * scale.  With
    ``sgate`` (float32 [T]) column ``experts`` of z is a gate logit: sgate = sigmoid of it."""
    _need(z, "z", torch.float32); _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32)
    T = z.shape[0]
    if ids.shape != (T, top) or weights.shape != (T, top) or (sgate is not None and (sgate.dtype != torch.float32 or sgate.numel() != T)):
        raise KernelError("moe_route: sizes do not fit")
    _ok(kernels().ce_moe_route(_ptr(z), _ptr(ids), _ptr(weights), _ptr(sgate), T, z.stride(0), int(experts), int(top), int(groups),
                               int(keep), float(scale), _stream()))


def moe_max_tiles(n_pairs: int, experts: int, tile: int) -> int:
    """The most tiles of ``tile`` rows that ``n_pairs`` (token, expert) pairs can fill when every expert's rows start a tile."""
    return n_pairs // tile + min(n_pairs, experts)


def moe_align(ids: torch.Tensor, experts: int, tile: int, row_token: torch.Tensor, pair_row: torch.Tensor,
              tile_expert: torch.Tensor, n_tiles: torch.Tensor) -> None:
    """Lay the pairs of ``ids`` [T, top] out by expert: ``row_token`` [rows] (the token of a row, -1 for padding),
    ``pair_row`` [T * top], ``tile_expert`` [tiles], ``n_tiles`` [1]; all int32 on the device."""
    for t, name in ((ids, "ids"), (row_token, "row_token"), (pair_row, "pair_row"), (tile_expert, "tile_expert"), (n_tiles, "n_tiles")):
        _need(t, name, torch.int32)
    n = ids.numel()
    if pair_row.numel() < n or tile_expert.numel() * tile > row_token.numel() or tile_expert.numel() < moe_max_tiles(n, experts, tile):
        raise KernelError("moe_align: the layout's tables are too small")
    _ok(kernels().ce_moe_align(_ptr(ids), n, ids.shape[1], int(experts), int(tile), row_token.numel(), _ptr(row_token),
                               _ptr(pair_row), _ptr(tile_expert), _ptr(n_tiles), _stream()))


def moe_matmul(inp: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile: int, activation: str = "none", row_token=None,
               tile_expert=None, n_tiles=None) -> None:
    """out[p] = act(inp[row_token[p]] @ w[tile_expert[p // tile]].T) for the rows of the layout's tiles (``row_token``
    None: the input rows are the layout's rows already).  Without any table: out = act(inp @ w[0].T), row by row.
    w [experts, N, K]; operands and output in one dtype."""
    _need(w, "w", inp.dtype); _need(out, "out", inp.dtype)
    if inp.stride(-1) != 1 or w.dim() != 3 or inp.shape[1] != w.shape[2] or out.shape[1] != w.shape[1]:
        raise KernelError("moe_matmul: shapes do not fit")
    if tile_expert is None:
        rows = inp.shape[0]
        tiles = (rows + tile - 1) // tile
        if out.shape[0] < rows:
            raise KernelError("moe_matmul: the output has fewer rows than the input")
    else:
        rows, tiles = out.shape[0], tile_expert.numel()
        if out.shape[0] < tiles * tile or (row_token is None and inp.shape[0] < tiles * tile):
            raise KernelError("moe_matmul: the layout has more rows than the operands")
    prof = profiling()
    if prof is not None:
        # what a step of this size moves and computes when every tile is full: the rows in and out, and the experts' weights
        # (each read once, at most as many as there are tiles)
        live = min(w.shape[0], max(tiles, 1))
        n_rows = min(rows, tiles * tile)
        prof.note_work((n_rows * (w.shape[1] + w.shape[2]) + live * w.shape[1] * w.shape[2]) * inp.element_size(),
                       2 * n_rows * w.shape[1] * w.shape[2])
    _ok(kernels().ce_moe_matmul(_ptr(inp), _ptr(w), _ptr(out), _ptr(row_token), _ptr(tile_expert), _ptr(n_tiles), dtype_code(inp.dtype),
                                tiles, int(tile), w.shape[1], w.shape[2], inp.stride(0), out.stride(0), MOE_ACTIVATIONS[activation],
                                rows, _stream()))


def moe_gather(inp: torch.Tensor, row_token: torch.Tensor, n_tiles: torch.Tensor, tile: int, out: torch.Tensor) -> None:
    """out[p] = inp[row_token[p]] (zeros where row_token[p] < 0) for the rows of the layout's live tiles; rows of whole
    16-byte pieces."""
    _need(out, "out", inp.dtype); _need(row_token, "row_token", torch.int32); _need(n_tiles, "n_tiles", torch.int32)
    if inp.stride(-1) != 1 or out.shape[1] != inp.shape[1] or row_token.numel() < out.shape[0]:
        raise KernelError("moe_gather: shapes do not fit")
    _ok(kernels().ce_moe_gather(_ptr(inp), inp.stride(0), inp.shape[1], inp.element_size(), _ptr(row_token), _ptr(n_tiles), int(tile),
                                _ptr(out), out.shape[0], _stream()))


def moe_combine(rows: torch.Tensor, pair_row: torch.Tensor, weights: torch.Tensor, y: torch.Tensor, shared=None, sgate=None,
                accumulate: bool = False) -> None:
    """y[t] (+)= sum_k weights[t, k] * rows[pair_row[t * top + k]] (+ sgate[t] * shared[t]); y float32 [T, W]."""
    _need(y, "y", torch.float32); _need(weights, "weights", torch.float32); _need(pair_row, "pair_row", torch.int32)
    T, top = weights.shape
    if y.shape[0] != T or rows.shape[1] != y.shape[1] or rows.stride(-1) != 1 or pair_row.numel() < T * top:
        raise KernelError("moe_combine: sizes do not fit")
    if shared is not None and (shared.dtype != rows.dtype or shared.shape != y.shape or not shared.is_contiguous()):
        raise KernelError("moe_combine: the shared expert's rows must be [T, W] in the experts' dtype")
    _ok(kernels().ce_moe_combine(_ptr(rows), dtype_code(rows.dtype), rows.stride(0), _ptr(pair_row), _ptr(weights), _ptr(shared),
                                 _ptr(sgate), _ptr(y), T, top, y.shape[1], 1 if accumulate else 0, _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    R, V = logits.shape
    _ok(kernels().ce_argmax(_ptr(logits), R, V, _ptr(out), _stream()))


SAMPLE_ROW = struct.Struct("<fffiQ")     # temperature, top_p, min_p, top_k, seed


def pack_sample_rows(rows: Sequence[tuple]) -> bytes:
    return b"".join(SAMPLE_ROW.pack(float(t), float(p), float(m), int(k), int(s) & 0xFFFFFFFFFFFFFFFF)
                    for (t, p, m, k, s) in rows)


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor) -> None:
    """params: uint8 [rows, 24] holding SAMPLE_ROW records."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32); _need(params, "params", torch.uint8)
    R, V = logits.shape
    if params.numel() != R * SAMPLE_ROW.size:
        raise KernelError("sample: params must hold one 24-byte record per row")
    _ok(kernels().ce_sample(_ptr(logits), R, V, _ptr(params), _ptr(out), _stream()))


def apply_penalties(logits: torch.Tensor, entries: torch.Tensor, row_params: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(entries, "entries", torch.int32)
    _need(row_params, "row_params", torch.float32)
    _ok(kernels().ce_apply_penalties(_ptr(logits), logits.shape[1], _ptr(entries), entries.shape[0],
                                     _ptr(row_params), _stream()))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.view(-1)[idx[i]] = val[i]"""
    _need(dst, "dst", torch.int32); _need(idx, "idx", torch.int32); _need(val, "val", torch.int32)
    _ok(kernels().ce_scatter_i32(_ptr(dst), _ptr(idx), _ptr(val), idx.numel(), dst.numel(), _stream()))
