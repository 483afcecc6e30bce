"""Loads libcarbon_kernels.so (built on first use) and declares the launchers' C interface.

There is no fallback: if the library cannot be built or loaded, importing an op raises.
"""
from __future__ import annotations

import ctypes
import threading

from . import build

_lib = None
_lock = threading.Lock()

_i, _f, _ll, _p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p

_SIGNATURES = {
    "ce_last_error": (ctypes.c_char_p, []),
    "ce_build_arch": (_i, []),
    "ce_kernel_counts": (_i, [ctypes.c_char_p, _i]),
    "ce_kernel_counts_reset": (None, []),
    "ce_last_kernel": (ctypes.c_char_p, []),
    "ce_set_pdl": (None, [_i]),
    # table, dtype, tokens, x, T, H, V, status, scale, stream
    "ce_embed": (_i, [_p, _i, _p, _p, _i, _i, _i, _p, _f, _p]),
    # x, w, out, out_dtype, rows, R, H, eps, stream
    "ce_rmsnorm": (_i, [_p, _p, _p, _i, _p, _i, _i, _f, _p]),
    # qkv, k_pool, v_pool, dtype, qw, kw, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
    # T, nh, nkv, d, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps, pairing, stream
    "ce_qk_rope_kvwrite": (_i, [_p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                                _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p]),
    "ce_add_residual": (_i, [_p, _p, _i, _ll, _p]),
    "ce_swiglu": (_i, [_p, _p, _i, _i, _i, _p]),
    "ce_reluglu": (_i, [_p, _p, _i, _i, _i, _p]),
    # in, out, dtype, T, I, ldo, stream
    "ce_relu2": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    # x, w, b, out, out_dtype, rows, R, H, eps, stream
    "ce_layernorm": (_i, [_p, _p, _p, _p, _i, _p, _i, _i, _f, _p]),
    # y, w, x, T, H, eps, stream
    "ce_rmsnorm_add": (_i, [_p, _p, _p, _p, _i, _i, _f, _p]),
    # x, n, cap, stream
    "ce_tanh_cap": (_i, [_p, _ll, _f, _p]),
    # src, out, out_dtype, T, ld, off, L, stream
    "ce_copy_cols": (_i, [_p, _p, _i, _i, _i, _i, _i, _p]),
    # z, table, dtype, tokens, out, T, D, ld, off, V, status, stream
    "ce_side_gate": (_i, [_p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p]),
    # rows, dtype, stride, off, n, first, first_stride, first_off, lam, T, stream
    "ce_value_mix": (_i, [_p, _i, _i, _i, _i, _p, _i, _i, _f, _i, _p]),
    # proj, wq, wkv, cq, k_pool, dtype, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
    # T, ld, off_q, qr, off_kv, r, dr, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps, stream
    "ce_latent_prepare": (_i, [_p] * 5 + [_i] + [_p] * 7 + [_i] * 13 + [_f, _p]),
    # src, src_stride, src_head, src_off, dst, dst_stride, dst_head, dst_off, dtype, cos, sin, positions, status,
    # T, H, dr, rd, max_pos, stream
    "ce_rope_part": (_i, [_p, _i, _i, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    # in, in_stride, in_head, W, out, out_stride, out_head, gate, gate_stride, gate_head, dtype, M, H, N, K, stream
    "ce_head_matmul": (_i, [_p, _i, _i, _p, _p, _i, _i, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    # q, k_pool, v_pool, gate, out, dtype, positions, seq_of_token, seq_slot, block_table, status, T, nh, nkv, d, dv,
    # q_stride, q_head, ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first, scale, softcap, sinks,
    # out_scale, stream
    "ce_masked_attention": (_i, [_p] * 5 + [_i] + [_p] * 5 + [_i] * 15 + [_f, _f, _p, _f, _p]),
    # proj, q_out, k_pool, v_pool, dtype, wq, wk, head_scale, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
    # T, ld, off_q, off_k, off_v, nh, nkv, d, dv, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps, stream
    "ce_norm_rope_kvwrite": (_i, [_p] * 4 + [_i] + [_p] * 10 + [_i] * 15 + [_f, _p]),
    # d, dv, q_stride, q_head, ldk, ldv, alias
    "ce_masked_attention_mma_supported": (_i, [_i] * 7),
    # q, k_pool, v_pool, gate, out, positions, seq_slot, q_start, block_table, tiles, status, n_tiles, n_tokens, nh, nkv, d, dv,
    # q_stride, q_head, ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first, scale, softcap, sinks,
    # out_scale, stream
    "ce_masked_attention_mma": (_i, [_p] * 11 + [_i] * 16 + [_f, _f, _p, _f, _p]),
    "ce_gated_delta_prep_width": (_i, [_i, _i, _i, _i]),
    # proj, dec, gz, taps, a_log, dt_bias, norm_w, prep, raw, state, kept, out, out_dtype, seq_of_token, seq_slot, q_start,
    # T, B, ld, off_conv, off_b, H, G, d, dv, K, eps, ld_dec, ld_gz, decay_mode, operands, rule, gate_act, out_scale,
    # cos, sin, positions, status, rd, max_pos, stage, stream
    "ce_gated_delta": (_i, [_p] * 12 + [_i] + [_p] * 3 + [_i] * 10 + [_f] + [_i] * 6 + [_f] + [_p] * 4 + [_i, _i, _i, _p]),
    # q, k_pool, v_pool, out, dtype, positions, seq_of_token, seq_slot, block_table, status,
    # T, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, stream
    "ce_attention_generic": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p,
                                  _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p]),
    # A, W, C, dtype, M, N, K, lda, ldc, mode, stream
    "ce_gemm_plain": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "ce_sample": (_i, [_p, _i, _i, _p, _p, _p]),
    "ce_argmax": (_i, [_p, _i, _i, _p, _p]),
    "ce_apply_penalties": (_i, [_p, _i, _p, _i, _p, _p]),
    "ce_scatter_i32": (_i, [_p, _p, _p, _i, _ll, _p]),
    # x, coef, w, out, out_dtype, rows, R, S, W, groups, eps, stream
    "ce_streams_norm": (_i, [_p, _p, _p, _p, _i, _p, _i, _i, _i, _i, _f, _p]),
    # h, mu, state, out, out_dtype, positions, seq_of_token, seq_slot, q_start, T, W, save, stream
    "ce_token_shift": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _p]),
    # h, state, seq_slot, q_start, B, W, stream
    "ce_save_last_rows": (_i, [_p, _p, _p, _p, _i, _i, _p]),
    # x, y, mix, c_out, bias, T, S, W, stream
    "ce_streams_write": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _p]),
    # x0, x, T, S, W, stream
    "ce_streams_broadcast": (_i, [_p, _p, _i, _i, _i, _p]),
    # out, dtype, bias, M, N, ld, stream
    "ce_add_bias": (_i, [_p, _i, _p, _i, _i, _i, _p]),
    # qkv, k_pool, v_pool, dtype, bias, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
    # T, stride, nq, nk, nv, d, dv, rd, page_size, max_pages, num_pages, max_pos, write_kv, stream
    "ce_bias_rope_kvwrite": (_i, [_p, _p, _p, _i] + [_p] * 8 + [_i] * 13 + [_p]),
    # q, k_pool, v_pool, gate, out, dtype, positions, seq_of_token, seq_slot, block_table, status, T, nh, nkv, d, dv,
    # q_stride, gate_stride, page_size, max_pages, num_pages, window, chunk, scale, lambda, eps, out_scale, stream
    "ce_diff_attention": (_i, [_p] * 5 + [_i] + [_p] * 5 + [_i] * 12 + [_f] * 4 + [_p]),
    "ce_diff_attention_mma_supported": (_i, [_i, _i, _i]),
    # q, k_pool, v_pool, gate, out, positions, seq_slot, q_start, block_table, tiles, status, n_tiles, nh, nkv, d, dv,
    # q_stride, gate_stride, page_size, max_pages, num_pages, window, chunk, scale, lambda, eps, out_scale, stream
    "ce_diff_attention_mma": (_i, [_p] * 11 + [_i] * 12 + [_f] * 4 + [_p]),
    # z, ids, weights, sgate, T, ld, E, top, groups, keep, scale, stream
    "ce_moe_route": (_i, [_p] * 4 + [_i] * 6 + [_f, _p]),
    "ce_moe_max_tiles": (_i, [_i, _i, _i]),
    # ids, n_pairs, top, E, BM, max_rows, row_token, pair_row, tile_expert, n_tiles, stream
    "ce_moe_align": (_i, [_p] + [_i] * 5 + [_p] * 5),
    # in, W, out, row_token, tile_expert, n_tiles, dtype, max_tiles, BM, N, K, ldi, ldo, act, n_rows, stream
    "ce_moe_matmul": (_i, [_p] * 6 + [_i] * 9 + [_p]),
    # in, ldi, K, elsize, row_token, n_tiles, BM, out, max_rows, stream
    "ce_moe_gather": (_i, [_p, _i, _i, _i, _p, _p, _i, _p, _i, _p]),
    # rows, dtype, ld, pair_row, weights, shared, sgate, y, T, top, W, accumulate, stream
    "ce_moe_combine": (_i, [_p, _i, _i] + [_p] * 5 + [_i] * 4 + [_p]),
    # proj, out, out_dtype, T, ld, off, L, stream
    "ce_tanh_cols": (_i, [_p, _p, _i, _i, _i, _i, _i, _p]),
    # proj, zz, w0, a_bias, norm_w, prep, raw, state, out, out_dtype, seq_slot, q_start, T, B, ld, off_r, off_k, off_v,
    # off_a, off_g, H, d, eps, stage, stream
    "ce_general_delta": (_i, [_p] * 9 + [_i] + [_p] * 2 + [_i] * 10 + [_f, _i, _p]),
}


class KernelError(RuntimeError):
    pass


def kernels() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            path = build.build_kernels()
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelError(f"cannot load the CUDA kernel library {path}: {exc}") from None
            for name, (res, args) in _SIGNATURES.items():
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    raise KernelError(f"{path} lacks the symbol {name}: rebuild the kernels") from None
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def declare(name: str, restype, argtypes) -> None:
    """Declare a launcher added by a later source file."""
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
