"""Python face of the CUDA launchers: argument checks, then one C call per kernel.

There is no other implementation behind these functions.  A tensor that is not on
a CUDA device, a missing library or a launch that the driver rejects raises
`KernelError`; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Callable, Dict, Optional

import torch

from . import build

MODE_STORE_F32 = 0
MODE_ACCUM_F32 = 1
MODE_SWIGLU = 2
MODE_STORE_ACT = 3
# what the tensor-core product's modes 2 and 3 can apply before rounding instead of their own operation
ACT_PLAIN, ACT_RELU_SQUARED, ACT_CLAMPED_GLU = 0, 1, 2

PAGE = build.PAGE_TOKENS  # tokens per cache page; the kernels are compiled with the same number


class KernelError(RuntimeError):
    pass


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_error_words: Dict[str, Callable[[], int]] = {}


def register_error_word(name: str, take: Callable[[], int]) -> None:
    """A kernel library whose waits are bounded names the function that reads and clears
    its error word (nonzero: a kernel gave up waiting, its results are not valid)."""
    _error_words[name] = take


def check_kernel_errors() -> None:
    """Reads every registered error word (this synchronises the device) and raises if one is
    set.  Callers use it where they wait for results anyway."""
    bad = {name: code for name, code in ((n, take()) for n, take in _error_words.items()) if code}
    if bad:
        raise KernelError("a kernel ran out of a bounded wait, its results are not valid: " +
                          ", ".join(f"{n}: code {c}" for n, c in bad.items()))
_counter = {"launches": 0}
_by_name: Dict[str, int] = {}


def launches() -> int:
    """Kernels launched through this module since the process started."""
    return _counter["launches"]


def launch_counts() -> Dict[str, int]:
    """The same count by launcher ("rmsnorm", "gemm_tc", "rope_cache_write", ...): what a
    test reads to see which kernels a step was made of."""
    return dict(_by_name)


def add_launches(n, sign: int = 1) -> None:
    """Counts kernels that ran without passing through this module: a replayed CUDA
    graph launches the kernels that were counted while it was recorded.  `n` is a number or
    a dictionary by launcher as `launch_counts` returns it."""
    if isinstance(n, dict):
        for k, v in n.items():
            _by_name[k] = _by_name.get(k, 0) + sign * v
        n = sum(n.values())
    _counter["launches"] += sign * n


def counts_since(before: Dict[str, int]) -> Dict[str, int]:
    """Launches by launcher since `before` (an earlier `launch_counts()`)."""
    return {k: v - before.get(k, 0) for k, v in _by_name.items() if v != before.get(k, 0)}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked of torch's C layer directly where it offers that: the Python
    `current_stream()` object costs some 15 us a call, a fifth of the host's time in a step launched
    kernel by kernel."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_sms: Dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _sms:
        _sms[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _sms[i]


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device; this package has no CPU path")
    return c_void_p(t.data_ptr())


def _check(status: int, what: str) -> None:
    _counter["launches"] += 1
    _by_name[what] = _by_name.get(what, 0) + 1
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if status == -2:
        raise KernelError(f"{what}: these sizes are not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _need(t: torch.Tensor, dtype: torch.dtype, what: str, contiguous: bool = True) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")


class CoreOps:
    """The kernels of one activation type (float32 or bfloat16)."""

    def __init__(self, act_dtype: torch.dtype):
        if act_dtype not in _SUFFIX:
            raise KernelError(f"no kernels for activation type {act_dtype}")
        self.act_dtype = act_dtype
        self.suffix = _SUFFIX[act_dtype]
        self.lib = build.load_library(f"core_{self.suffix}")
        for base in ("tl_embed", "tl_softcap", "tl_advance_step", "tl_regroup_step", "tl_convert", "tl_rmsnorm", "tl_rope_cache_write", "tl_silu_mul",
                     "tl_gemm_generic", "tl_attn_generic", "tl_pair_embed_add", "tl_branch_norm_add", "tl_poly_norm",
                     "tl_latent_prep", "tl_headwise_gemm", "tl_latent_attn", "tl_gated_scan", "tl_gated_scan_groups",
                     "tl_stream_spread", "tl_stream_sum", "tl_hc_read_norm", "tl_hc_write", "tl_branch_norm_mean",
                     "tl_headnorm_silu_gate", "tl_qk_norm_cache_write", "tl_sink_attn", "tl_gla_scan", "tl_gla_scan_scratch",
                     "tl_moe_route", "tl_moe_plan", "tl_moe_gemm", "tl_moe_combine", "tl_moe_route_grouped",
                     "tl_rotary_cache_write", "tl_diff_heads", "tl_sigmoid_gate", "tl_norm_add_norm", "tl_relu_squared",
                     "tl_clamped_glu", "tl_delta_prep", "tl_conv_state_update", "tl_delta_scan", "tl_silu_rows",
                     "tl_weighted_sum"):
            fn = getattr(self.lib, f"{base}_{self.suffix}")
            fn.restype = c_int
            setattr(self, "_" + base, fn)

    # x[t, :] = table[tokens[t], :]
    def embed(self, tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor,
              token_from: Optional[torch.Tensor] = None,
              token_src: Optional[torch.Tensor] = None, scale: float = 1.0,
              position_table: Optional[torch.Tensor] = None,
              token_pos: Optional[torch.Tensor] = None) -> None:
        """x[t] = scale * table[token t] (+ position_table[token_pos[t]]).  With `token_src`
        (int32 on the device), token t is token_src[token_from[t]] wherever token_from[t] >= 0,
        else tokens[t]."""
        _need(tokens, torch.int32, "embed tokens")
        _need(table, self.act_dtype, "embed table")
        _need(x, torch.float32, "embed out")
        if token_src is not None:
            _need(token_src, torch.int32, "embed token source")
            _need(token_from, torch.int32, "embed token index")
        T, H = x.shape
        max_pos = 0
        if position_table is not None:
            _need(position_table, self.act_dtype, "embed position table")
            _need(token_pos, torch.int32, "embed token positions")
            if position_table.shape[1] != H:
                raise KernelError("embed: the position table's width is not the stream's")
            max_pos = position_table.shape[0]
        _check(self._tl_embed(_ptr(tokens), _ptr(token_from if token_src is not None else None),
                              _ptr(token_src), _ptr(table), _ptr(x), c_int(T), c_int(H),
                              c_int(table.shape[0]), c_float(scale), _ptr(position_table),
                              _ptr(token_pos if position_table is not None else None), c_int(max_pos),
                              _stream()), "embed")

    def convert_into(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """dst (activation type, contiguous, on the device) = src (32-bit, bfloat16 or float16, the
        same number of elements, contiguous, on the device): a weight on its way into the model."""
        kinds = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
        if src.dtype not in kinds:
            raise KernelError(f"convert: unsupported stored type {src.dtype}")
        _need(dst, self.act_dtype, "convert destination")
        if not src.is_contiguous() or src.numel() != dst.numel():
            raise KernelError("convert: source and destination must be contiguous and of one size")
        from ctypes import c_longlong
        _check(self._tl_convert(_ptr(src), c_int(kinds[src.dtype]), _ptr(dst), c_longlong(dst.numel()), _stream()),
               "convert")

    def advance_step(self, token_pos: torch.Tensor, seq_len: torch.Tensor) -> None:
        """Every row's position and length go up by one, on the device (a decode step of the same
        batch as the step before)."""
        _need(token_pos, torch.int32, "advance positions")
        _need(seq_len, torch.int32, "advance lengths")
        if token_pos.numel() != seq_len.numel():
            raise KernelError("advance_step: one position and one length per row are needed")
        _check(self._tl_advance_step(_ptr(token_pos), _ptr(seq_len), c_int(seq_len.numel()), _stream()),
               "advance_step")

    REGROUP_MAX_ROWS = 256

    def regroup_step(self, old_pos: torch.Tensor, old_len: torch.Tensor, old_slot: torch.Tensor,
                     base: torch.Tensor, offsets, keep, token_from) -> None:
        """The arrays of a decode step of the rows `keep` of the decode step before (whose positions,
        lengths and slots are `old_*`), written into `base` at `offsets` (eight starts, in the order
        tokens, token_seq, token_pos, seq_slot, seq_start, seq_len, want_rows, token_from); row j takes
        its token from place token_from[j] of the sampler's output.  The old arrays may lie in `base`."""
        from ctypes import c_ushort
        n = len(keep)
        if n > self.REGROUP_MAX_ROWS or len(token_from) != n or len(offsets) != 8:
            raise KernelError("regroup_step: at most 256 rows, one source place per row, eight offsets")
        if n and (max(keep) >= old_pos.numel() or max(keep) > 65535 or max(token_from) > 65535
                  or min(keep) < 0 or min(token_from) < 0):
            raise KernelError("regroup_step: a row or a source place is out of range")
        for t, what in ((old_pos, "positions"), (old_len, "lengths"), (old_slot, "slots"), (base, "buffer")):
            _need(t, torch.int32, "regroup " + what)
        if max(offsets) + n + 1 > base.numel():
            raise KernelError("regroup_step: the new layout does not fit the buffer")
        _check(self._tl_regroup_step(_ptr(old_pos), _ptr(old_len), _ptr(old_slot), _ptr(base),
                                     (c_int * 8)(*[int(o) for o in offsets]), c_int(n),
                                     (c_ushort * max(n, 1))(*[int(k) for k in keep]),
                                     (c_ushort * max(n, 1))(*[int(f) for f in token_from]), _stream()),
               "regroup_step")

    def softcap(self, logits: torch.Tensor, cap: float) -> None:
        """logits <- cap * tanh(logits / cap), in place."""
        _need(logits, torch.float32, "softcap logits")
        from ctypes import c_longlong
        _check(self._tl_softcap(_ptr(logits), c_longlong(logits.numel()), c_float(cap), _stream()),
               "softcap")

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        _need(x, torch.float32, "rmsnorm in")
        _need(out, self.act_dtype, "rmsnorm out")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"rmsnorm weight: unsupported dtype {weight.dtype}")
        n_rows, H = out.shape
        if weight.numel() != H or x.shape[1] != H:
            raise KernelError("rmsnorm: sizes do not match")
        if rows is not None:
            _need(rows, torch.int32, "rmsnorm rows")
        _check(self._tl_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight),
                                c_int(1 if weight.dtype == torch.float32 else 0), _ptr(out),
                                c_int(n_rows), c_int(H), c_float(eps), _stream()), "rmsnorm")

    def rope_cache_write(self, qkv: torch.Tensor, q_out: torch.Tensor,
                         k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                         token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                         page_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                         style: int, nh: int, nkv: int, hd: int) -> None:
        _need(qkv, torch.float32, "rope qkv")
        _need(q_out, self.act_dtype, "rope q out")
        T = qkv.shape[0]
        stride = 0
        if k_pages is not None:
            _need(k_pages, self.act_dtype, "k pages")
            _need(v_pages, self.act_dtype, "v pages")
            _need(page_table, torch.int32, "page table")
            stride = page_table.stride(0)
            if qkv.shape[1] < (nh + 2 * nkv) * hd:
                raise KernelError("rope: qkv has too few columns")
        if inv_freq is not None:
            _need(inv_freq, torch.float32, "inv_freq")
            if inv_freq.numel() != hd // 2:
                raise KernelError("rope: inv_freq must have head_dim/2 entries")
        _check(self._tl_rope_cache_write(
            _ptr(qkv), c_int(qkv.stride(0)), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
            _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), c_int(stride),
            _ptr(inv_freq), c_int(style), c_int(T), c_int(nh), c_int(nkv), c_int(hd), _stream()),
            "rope_cache_write")

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor) -> None:
        _need(gu, torch.float32, "silu_mul in")
        _need(out, self.act_dtype, "silu_mul out")
        T, I = out.shape
        _check(self._tl_silu_mul(_ptr(gu), _ptr(out), c_int(T), c_int(I), _stream()), "silu_mul")

    def gemm_generic(self, a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, mode: int) -> None:
        """c (op)= a @ w.T; in SwiGLU mode w holds the gate rows, then the up rows."""
        _need(a, self.act_dtype, "gemm a", contiguous=False)
        _need(w, self.act_dtype, "gemm w", contiguous=False)
        want_c = torch.float32 if mode in (MODE_STORE_F32, MODE_ACCUM_F32) else self.act_dtype
        _need(c, want_c, "gemm c", contiguous=False)
        M, K = a.shape
        N = c.shape[1]
        rows_w = 2 * N if mode == MODE_SWIGLU else N
        if w.shape != (rows_w, K) or c.shape[0] != M:
            raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)} w {tuple(w.shape)} "
                              f"c {tuple(c.shape)} mode {mode}")
        if a.stride(1) != 1 or w.stride(1) != 1 or c.stride(1) != 1:
            raise KernelError("gemm: the last dimension must be contiguous")
        _check(self._tl_gemm_generic(_ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)),
                                     _ptr(c), c_int(c.stride(0)), c_int(M), c_int(N), c_int(K),
                                     c_int(mode), _stream()), "gemm_generic")

    def attn_generic(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     out: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                     seq_slot: torch.Tensor, page_table: torch.Tensor, nh: int, nkv: int, hd: int,
                     window: Optional[int], scale: float) -> None:
        for t, n in ((q, "attn q"), (k_pages, "k pages"), (v_pages, "v pages"), (out, "attn out")):
            _need(t, self.act_dtype, n)
        _need(page_table, torch.int32, "page table")
        T = q.shape[0]
        _check(self._tl_attn_generic(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(token_pos), _ptr(token_seq),
            _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), c_int(T), c_int(nh),
            c_int(nkv), c_int(hd), c_int(window or 0), c_float(scale), _stream()), "attn_generic")

    # ---- sublayers that read the stream itself, with the norm on their output -------------------
    def pair_embed_add(self, batch_tokens: torch.Tensor, token_from: Optional[torch.Tensor],
                       token_src: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
                       seq_slot: torch.Tensor, seq_start: torch.Tensor, last_token: torch.Tensor,
                       table: torch.Tensor, x: torch.Tensor, vocab: int, buckets: int, mul_prev: int,
                       mul_cur: int) -> None:
        """x[t] += table[(prev * mul_prev + token * mul_cur) mod buckets], the table's last row for a
        sequence's first token; `last_token` ([slots] int32) holds every sequence's latest token and is
        brought up to date (a second kernel)."""
        from ctypes import c_longlong
        _need(table, self.act_dtype, "pair table")
        _need(x, torch.float32, "pair embed stream")
        _need(last_token, torch.int32, "last tokens")
        T, H = x.shape
        if table.shape != (buckets + 1, H):
            raise KernelError("pair_embed_add: the table must have buckets + 1 rows of the stream's width")
        _check(self._tl_pair_embed_add(
            _ptr(batch_tokens), _ptr(token_from if token_src is not None else None), _ptr(token_src),
            _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(seq_start), _ptr(last_token), _ptr(table),
            _ptr(x), c_int(T), c_int(seq_slot.numel()), c_int(H), c_int(vocab), c_int(buckets),
            c_longlong(mul_prev), c_longlong(mul_cur), _stream()), "pair_embed_add")
        _check(0, "remember_last_token")

    def branch_norm_add(self, y: torch.Tensor, gain: torch.Tensor, mult: float, eps: float, x: torch.Tensor,
                        xb: Optional[torch.Tensor] = None) -> None:
        """x += mult * gain * y / rms(y), row by row, `gain` one 32-bit number on the device; `xb`
        (activation type) also receives the new x."""
        _need(y, torch.float32, "branch output", contiguous=False)
        _need(x, torch.float32, "stream")
        _need(gain, torch.float32, "branch gain")
        rows, H = x.shape
        if y.shape != x.shape or y.stride(1) != 1 or gain.numel() != 1:
            raise KernelError("branch_norm_add: sizes do not match")
        if xb is not None:
            _need(xb, self.act_dtype, "stream copy")
        _check(self._tl_branch_norm_add(_ptr(y), c_int(y.stride(0)), _ptr(gain), c_float(mult), c_float(eps),
                                        _ptr(x), _ptr(xb), c_int(rows), c_int(H), _stream()), "branch_norm_add")

    def poly_norm(self, z: torch.Tensor, coeff: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """out = a N(z) + b N(z^2) + c N(z^3) + e per row, coeff = (a, b, c, e) 32-bit on the device."""
        _need(z, torch.float32, "poly_norm in", contiguous=False)
        _need(out, self.act_dtype, "poly_norm out")
        _need(coeff, torch.float32, "poly_norm coefficients")
        rows, F = out.shape
        if z.shape != out.shape or z.stride(1) != 1 or coeff.numel() != 4:
            raise KernelError("poly_norm: sizes do not match")
        _check(self._tl_poly_norm(_ptr(z), c_int(z.stride(0)), _ptr(coeff), c_float(eps), _ptr(out), c_int(rows),
                                  c_int(F), _stream()), "poly_norm")

    # ---- attention through latents ----------------------------------------------------------------
    def latent_prep(self, dq: torch.Tensor, dkv: torch.Tensor, wq: torch.Tensor, wc: torch.Tensor, eps: float,
                    cq: torch.Tensor, pages: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                    seq_slot: torch.Tensor, page_table: torch.Tensor, inv_freq: Optional[torch.Tensor],
                    rank: int, rot: int, dims: int) -> None:
        """cq = norm(dq) * wq; the token's page row = [norm(dkv[:, :rank]) * wc | rotate(dkv[:, rank:])]."""
        for t, n in ((dq, "query down-projection"), (dkv, "key/value down-projection")):
            _need(t, torch.float32, n, contiguous=False)
            if t.stride(1) != 1:
                raise KernelError(f"latent_prep: {n} must have contiguous rows")
        _need(wq, torch.float32, "query latent norm weight")
        _need(wc, torch.float32, "latent norm weight")
        _need(cq, self.act_dtype, "query latent")
        _need(pages, self.act_dtype, "latent pages")
        _need(page_table, torch.int32, "page table")
        T, q_rank = cq.shape
        if dq.shape != (T, q_rank) or dkv.shape != (T, rank + rot) or wq.numel() != q_rank or \
                wc.numel() != rank or pages.shape[1:] != (PAGE, rank + rot):
            raise KernelError("latent_prep: sizes do not match")
        if dims:
            _need(inv_freq, torch.float32, "inv_freq")
            if inv_freq.numel() != dims // 2:
                raise KernelError("latent_prep: inv_freq must have dims/2 entries")
        _check(self._tl_latent_prep(
            _ptr(dq), c_int(dq.stride(0)), _ptr(dkv), c_int(dkv.stride(0)), _ptr(wq), _ptr(wc), c_float(eps),
            _ptr(cq), _ptr(pages), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table),
            c_int(page_table.stride(0)), _ptr(inv_freq if dims else None), c_int(T), c_int(q_rank), c_int(rank),
            c_int(rot), c_int(dims), _stream()), "latent_prep")

    def headwise_gemm(self, a: torch.Tensor, a_head: int, w: torch.Tensor, c: torch.Tensor, c_head: int,
                      gate: Optional[torch.Tensor] = None, act_out: bool = False) -> None:
        """c[t, h * c_head + n] = sum_k a[t, h * a_head + k] * w[h, n, k] for every head h; with `gate`
        ([T, heads * N] 32-bit) the result is multiplied by sigmoid(gate) and `c` is of the activation
        type; without a gate `c` is 32-bit, or, with `act_out`, of the activation type."""
        act_out = act_out or gate is not None
        _need(a, torch.float32, "headwise a", contiguous=False)
        _need(w, self.act_dtype, "headwise w")
        _need(c, self.act_dtype if act_out else torch.float32, "headwise c", contiguous=False)
        heads, N, K = w.shape
        M = a.shape[0]
        if a.stride(1) != 1 or c.stride(1) != 1 or c.shape[0] != M or \
                a.shape[1] < (heads - 1) * a_head + K or c.shape[1] < (heads - 1) * c_head + N:
            raise KernelError("headwise_gemm: sizes do not match")
        ldg = 0
        if gate is not None:
            _need(gate, torch.float32, "headwise gate", contiguous=False)
            if gate.shape != (M, heads * N) or gate.stride(1) != 1:
                raise KernelError("headwise_gemm: the gate must be [rows, heads * outputs]")
            ldg = gate.stride(0)
        if act_out and M > 16 and self.act_dtype == torch.bfloat16:
            # many rows: the tensor-core kernel, where sizes and alignments allow it
            self.lib.tl_headwise_mma.restype = c_int
            st = self.lib.tl_headwise_mma(_ptr(a), c_int(a.stride(0)), c_int(a_head), _ptr(w), _ptr(c),
                                          c_int(c.stride(0)), c_int(c_head), _ptr(gate), c_int(ldg), c_int(M),
                                          c_int(N), c_int(K), c_int(heads), _stream())
            if st != -2:
                _check(st, "headwise_mma")
                return
        _check(self._tl_headwise_gemm(_ptr(a), c_int(a.stride(0)), c_int(a_head), _ptr(w), _ptr(c),
                                      c_int(c.stride(0)), c_int(c_head), _ptr(gate), c_int(ldg), c_int(M), c_int(N),
                                      c_int(K), c_int(heads), c_int(1 if act_out else 0), _stream()),
               "headwise_gemm")

    def latent_attn(self, qa: torch.Tensor, qa_head: int, q: torch.Tensor, q_head: int, q_off: int,
                    pages: torch.Tensor, out: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                    seq_slot: torch.Tensor, page_table: torch.Tensor, inv_freq: Optional[torch.Tensor], heads: int,
                    rank: int, rot: int, dims: int, window: Optional[int], scale: float,
                    max_keys: Optional[int] = None, workspace=None, sink: Optional[torch.Tensor] = None) -> None:
        """out[t, h, :] = softmax over the visible positions of ((qa[t, h] . c + rotate(q_rot[t, h]) . r) *
        scale) times the positions' c; page rows are [c | r].  Head h's latent-space query starts at column
        h * qa_head of `qa`, its part to rotate at column h * q_head + q_off of `q` (one buffer may be both).

        In bfloat16 the tensor-core kernel runs where the sizes allow it (rank and rot multiples of 16,
        rank <= 512); `max_keys` (an upper bound of the keys a token of the step sees) lets it cut the keys
        of a step of few tokens into parts, whose partial sums lie in a buffer of `workspace`.  `sink` (one
        32-bit number per head) adds exp(sink[h]) to the softmax's denominator, once."""
        if sink is not None:
            _need(sink, torch.float32, "sink")
            if sink.numel() != heads:
                raise KernelError("latent_attn: one sink per head is needed")
        _need(qa, torch.float32, "latent queries", contiguous=False)
        _need(q, torch.float32, "queries", contiguous=False)
        _need(pages, self.act_dtype, "latent pages")
        _need(out, torch.float32, "latent attention out")
        _need(page_table, torch.int32, "page table")
        T = qa.shape[0]
        if out.shape != (T, heads, rank) or q.stride(1) != 1 or qa.stride(1) != 1 or q.shape[0] != T or \
                pages.shape[1:] != (PAGE, rank + rot) or q.shape[1] < (heads - 1) * q_head + q_off + rot or \
                qa.shape[1] < (heads - 1) * qa_head + rank:
            raise KernelError("latent_attn: sizes do not match")
        if self.act_dtype == torch.bfloat16:
            from ctypes import byref, c_longlong
            n = c_longlong(0)
            bound = min(int(max_keys), int(window)) if (max_keys and window) else int(max_keys or window or (1 << 30))
            splits = self.lib.tl_latent_attn_plan(c_int(T), c_int(heads), c_int(rank), c_int(rot), c_int(bound),
                                                  c_int(_sm_count(qa.device)), byref(n))
            if splits >= 1:
                part = None
                if n.value:
                    part = (workspace.get("latent_attn_parts", (n.value,), torch.float32) if workspace is not None
                            else torch.empty(n.value, dtype=torch.float32, device=qa.device))
                self.lib.tl_latent_attn_mma.restype = c_int
                _check(self.lib.tl_latent_attn_mma(
                    _ptr(qa), c_int(qa.stride(0)), c_int(qa_head), _ptr(q), c_int(q.stride(0)), c_int(q_head),
                    c_int(q_off), _ptr(pages), _ptr(out), _ptr(part), _ptr(token_pos), _ptr(token_seq),
                    _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), _ptr(inv_freq if dims else None),
                    _ptr(sink), c_int(T), c_int(heads), c_int(rank), c_int(rot), c_int(dims), c_int(window or 0),
                    c_float(scale), c_int(splits), _stream()), "latent_attn_mma")
                if splits > 1:
                    _check(0, "latent_attn_merge")
                return
        _check(self._tl_latent_attn(
            _ptr(qa), c_int(qa.stride(0)), c_int(qa_head), _ptr(q), c_int(q.stride(0)), c_int(q_head), c_int(q_off),
            _ptr(pages), _ptr(out), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table),
            c_int(page_table.stride(0)), _ptr(inv_freq if dims else None), _ptr(sink), c_int(T), c_int(heads),
            c_int(rank), c_int(rot), c_int(dims), c_int(window or 0), c_float(scale), _stream()), "latent_attn")

    # ---- gated linear recurrence ------------------------------------------------------------------
    def gated_scan(self, z: torch.Tensor, bias: torch.Tensor, low: torch.Tensor, state: torch.Tensor,
                   out: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor, heads: int, dim: int,
                   vdim: int, workspace=None) -> None:
        """The recurrence S <- diag(f) S + (1 - f) v^T, o = S^T q over each sequence's tokens of the step,
        from and into `state` [slots, heads, dim, vdim]; `z` [T, 2 heads dim + heads vdim] 32-bit holds the
        projections for q, f and v side by side (for steps of many tokens per sequence the q and f columns
        are overwritten with their activations)."""
        _need(z, torch.float32, "recurrence projections", contiguous=False)
        for t, n in ((bias, "forget bias"), (low, "forget lower bound"), (state, "recurrent state"),
                     (out, "recurrence out")):
            _need(t, torch.float32, n)
        T = z.shape[0]
        hd = heads * dim
        if z.shape[1] != 2 * hd + heads * vdim or z.stride(1) != 1 or out.shape != (T, heads * vdim) or \
                bias.numel() != hd or low.numel() != hd or state.shape[1:] != (heads, dim, vdim):
            raise KernelError("gated_scan: sizes do not match")
        # long steps: the state's rows are shared out over several warps, whose sums are added afterwards
        groups = self._tl_gated_scan_groups(c_int(T), c_int(seq_slot.numel()), c_int(dim))
        slices = None
        if groups > 1:
            n = groups * T * heads * vdim
            slices = (workspace.get("scan_slices", (n,), torch.float32) if workspace is not None
                      else torch.empty(n, dtype=torch.float32, device=z.device))
        _check(self._tl_gated_scan(_ptr(z), _ptr(z[:, hd:]), _ptr(z[:, 2 * hd:]), c_int(z.stride(0)), _ptr(bias),
                                   _ptr(low), _ptr(state), _ptr(out), c_int(out.stride(0)), _ptr(seq_start),
                                   _ptr(seq_slot), c_int(T), c_int(seq_slot.numel()), c_int(heads), c_int(dim),
                                   c_int(vdim), _ptr(slices), _stream()), "gated_scan")
        if T > 4 * seq_slot.numel():
            _check(0, "scan_gates")
        if groups > 1:
            _check(0, "scan_sum_slices")

    # ---- several residual streams (hyper-connections) ---------------------------------------------
    def stream_spread(self, x: torch.Tensor, xs: torch.Tensor) -> None:
        """xs[t, s, :] = x[t, :] for every stream s."""
        _need(x, torch.float32, "stream")
        _need(xs, torch.float32, "streams")
        T, S, H = xs.shape
        if x.shape != (T, H):
            raise KernelError("stream_spread: sizes do not match")
        _check(self._tl_stream_spread(_ptr(x), _ptr(xs), c_int(T), c_int(H), c_int(S), _stream()), "stream_spread")

    def stream_sum(self, xs: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        """x[r, :] = sum_s xs[rows[r], s, :] (all rows in order without `rows`)."""
        _need(x, torch.float32, "stream")
        _need(xs, torch.float32, "streams")
        _, S, H = xs.shape
        if x.shape[1] != H:
            raise KernelError("stream_sum: sizes do not match")
        if rows is not None:
            _need(rows, torch.int32, "stream_sum rows")
        _check(self._tl_stream_sum(_ptr(xs), _ptr(rows), _ptr(x), c_int(x.shape[0]), c_int(H), c_int(S), _stream()),
               "stream_sum")

    def hc_read_norm(self, xs: torch.Tensor, a: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """out[t] = act(u / rms(u) * w) with u = sum_s a[s] xs[t, s]; `w` 32-bit per coordinate."""
        _need(xs, torch.float32, "streams")
        _need(a, torch.float32, "stream read weights")
        _need(w, torch.float32, "norm factor")
        _need(out, self.act_dtype, "normed input")
        T, S, H = xs.shape
        if a.numel() != S or w.numel() != H or out.shape != (T, H):
            raise KernelError("hc_read_norm: sizes do not match")
        _check(self._tl_hc_read_norm(_ptr(xs), _ptr(a), _ptr(w), c_float(eps), _ptr(out), c_int(T), c_int(H),
                                     c_int(S), _stream()), "hc_read_norm")

    def hc_write(self, xs: torch.Tensor, mix: torch.Tensor, b: torch.Tensor, y: torch.Tensor,
                 next_read=None) -> None:
        """xs'[t, j] = sum_s mix[s, j] xs[t, s] + b[j] y[t], in place.  `next_read` = (a, w, eps, out): the
        kernel also does the next sublayer's read and norm (see `hc_read_norm`) on the new streams."""
        _need(xs, torch.float32, "streams")
        _need(mix, torch.float32, "stream mix")
        _need(b, torch.float32, "stream write weights")
        _need(y, torch.float32, "sublayer output", contiguous=False)
        T, S, H = xs.shape
        if mix.shape != (S, S) or b.numel() != S or y.shape != (T, H) or y.stride(1) != 1:
            raise KernelError("hc_write: sizes do not match")
        a2 = w2 = out2 = None
        eps2 = 0.0
        if next_read is not None:
            a2, w2, eps2, out2 = next_read
            _need(a2, torch.float32, "stream read weights")
            _need(w2, torch.float32, "norm factor")
            _need(out2, self.act_dtype, "normed input")
            if a2.numel() != S or w2.numel() != H or out2.shape != (T, H):
                raise KernelError("hc_write: sizes of the next read do not match")
        _check(self._tl_hc_write(_ptr(xs), _ptr(mix), _ptr(b), _ptr(y), c_int(y.stride(0)), c_int(T), c_int(H),
                                 c_int(S), _ptr(a2), _ptr(w2), c_float(eps2), _ptr(out2), _stream()), "hc_write")

    def branch_norm_mean(self, ys, ws, eps: float, out: torch.Tensor, accumulate: bool) -> None:
        """out (+)= mean over the branches of y_b / rms(y_b) * w_b, row by row (up to 4 branches)."""
        _need(out, torch.float32, "mixer output")
        T, H = out.shape
        for y, w in zip(ys, ws):
            _need(y, torch.float32, "branch output")
            _need(w, torch.float32, "branch norm weight")
            if y.shape != (T, H) or w.numel() != H:
                raise KernelError("branch_norm_mean: sizes do not match")
        n = len(ys)
        yp = (c_void_p * n)(*[y.data_ptr() for y in ys])
        wp = (c_void_p * n)(*[w.data_ptr() for w in ws])
        _check(self._tl_branch_norm_mean(yp, wp, c_int(n), c_int(T), c_int(H), c_float(eps), _ptr(out),
                                         c_int(1 if accumulate else 0), _stream()), "branch_norm_mean")

    def headnorm_silu_gate(self, o: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor,
                           out: torch.Tensor, heads: int, vdim: int, sigmoid: bool = False) -> None:
        """out[t, h] = act(o[t, h] / rms(o[t, h]) * w * silu(gate[t, h])), the norm over a head's entries;
        with `sigmoid` the gate's function is the sigmoid.  One head of the whole width norms the
        concatenated heads together."""
        _need(o, torch.float32, "head outputs")
        _need(w, torch.float32, "head norm weight")
        _need(gate, torch.float32, "gate", contiguous=False)
        _need(out, self.act_dtype, "gated output")
        T = o.shape[0]
        if o.shape != (T, heads * vdim) or out.shape != o.shape or gate.shape != o.shape or gate.stride(1) != 1 or \
                w.numel() != vdim:
            raise KernelError("headnorm_silu_gate: sizes do not match")
        _check(self._tl_headnorm_silu_gate(_ptr(o), _ptr(w), c_float(eps), _ptr(gate), c_int(gate.stride(0)),
                                           _ptr(out), c_int(T), c_int(heads), c_int(vdim),
                                           c_int(1 if sigmoid else 0), _stream()),
               "headnorm_silu_gate")

    # ---- attention with a sink, capped scores and a window that keeps the first keys --------------
    def qk_norm_cache_write(self, z: torch.Tensor, bias: Optional[torch.Tensor], qw: Optional[torch.Tensor],
                            kw: Optional[torch.Tensor], eps: float, q_out: torch.Tensor, k_pages: torch.Tensor,
                            v_pages: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                            seq_slot: torch.Tensor, page_table: torch.Tensor, nh: int, nkv: int, dim: int,
                            vdim: int) -> None:
        """The projections `z` (32-bit rows: q heads, k heads, v heads) get `bias`; q and k are RMS-normed per
        head with the weights `qw` / `kw` (None: no norm); q goes to `q_out`, k and v into the pages."""
        _need(z, torch.float32, "projections", contiguous=False)
        _need(q_out, self.act_dtype, "q out")
        _need(k_pages, self.act_dtype, "k pages")
        _need(v_pages, self.act_dtype, "v pages")
        _need(page_table, torch.int32, "page table")
        T = z.shape[0]
        cols = (nh + nkv) * dim + nkv * vdim
        if z.shape[1] < cols or z.stride(1) != 1 or q_out.shape != (T, nh * dim) or \
                k_pages.shape[1:] != (nkv, PAGE, dim) or v_pages.shape[1:] != (nkv, vdim, PAGE):
            raise KernelError("qk_norm_cache_write: sizes do not match")
        for t, n, what in ((bias, cols, "bias"), (qw, dim, "q norm weight"), (kw, dim, "k norm weight")):
            if t is not None:
                _need(t, torch.float32, what)
                if t.numel() != n:
                    raise KernelError(f"qk_norm_cache_write: {what} must have {n} entries")
        _check(self._tl_qk_norm_cache_write(
            _ptr(z), c_int(z.stride(0)), _ptr(bias), _ptr(qw), _ptr(kw), c_float(eps), _ptr(q_out), _ptr(k_pages),
            _ptr(v_pages), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table),
            c_int(page_table.stride(0)), c_int(T), c_int(nh), c_int(nkv), c_int(dim), c_int(vdim), _stream()),
            "qk_norm_cache_write")

    def sink_attn(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, gate: Optional[torch.Tensor],
                  sink: Optional[torch.Tensor], out: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                  seq_slot: torch.Tensor, page_table: torch.Tensor, nh: int, nkv: int, dim: int, vdim: int,
                  window: Optional[int], keep_first: int, scale: float, softcap: Optional[float]) -> None:
        """out[t, h] = sigmoid(gate[t, h]) * sum_j p_j v_j over the visible keys j (j <= i and (i - j < window
        or j < keep_first)), scores capped by `softcap`, the softmax's denominator also holding exp(sink[h])."""
        for t, n in ((q, "attn q"), (k_pages, "k pages"), (v_pages, "v pages"), (out, "attn out")):
            _need(t, self.act_dtype, n)
        _need(page_table, torch.int32, "page table")
        T = q.shape[0]
        if q.shape != (T, nh * dim) or out.shape != (T, nh * vdim) or k_pages.shape[1:] != (nkv, PAGE, dim) or \
                v_pages.shape[1:] != (nkv, vdim, PAGE):
            raise KernelError("sink_attn: sizes do not match")
        ldg = 0
        if gate is not None:
            _need(gate, torch.float32, "head gate", contiguous=False)
            if gate.shape != (T, nh) or gate.stride(1) != 1:
                raise KernelError("sink_attn: the gate must be [tokens, heads]")
            ldg = gate.stride(0)
        if sink is not None:
            _need(sink, torch.float32, "sink")
            if sink.numel() != nh:
                raise KernelError("sink_attn: one sink per head is needed")
        _check(self._tl_sink_attn(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(gate), c_int(ldg), _ptr(sink), _ptr(out), _ptr(token_pos),
            _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), c_int(T), c_int(nh),
            c_int(nkv), c_int(dim), c_int(vdim), c_int(window or 0), c_int(keep_first or 0), c_float(scale),
            c_float(softcap or 0.0), _stream()), "sink_attn")

    # ---- gated linear attention ---------------------------------------------------------------------
    def gla_scan(self, zq: torch.Tensor, zk: torch.Tensor, zv: torch.Tensor, za: torch.Tensor,
                 bias: Optional[torch.Tensor], tau: float, q_scale: float, state: torch.Tensor, out: torch.Tensor,
                 seq_start: torch.Tensor, seq_slot: torch.Tensor, heads: int, dim: int, vdim: int,
                 workspace=None, chunked: bool = True, given: bool = False) -> None:
        """S <- diag(alpha) S + k v^T, o = S^T (q * q_scale) over each sequence's tokens of the step, from and
        into `state` [slots, heads, dim, vdim]; alpha = sigmoid(za + bias)^(1 / tau).  zq, zk, zv are column
        ranges of one 32-bit product (one row stride); `za` may be overwritten with the decays.  Long steps
        run in three passes over chunks of 64 tokens (`chunked`; the same sums in another order), with
        scratch from `workspace`.  With `given`, `za` holds the decays themselves and is only read; it may
        then be one row [1, heads * dim] that serves every token (a decay that is a constant of the head)."""
        for t, n in ((zq, "q"), (zk, "k"), (zv, "v"), (za, "decay pre-activations")):
            _need(t, torch.float32, "recurrence " + n, contiguous=False)
            if t.stride(1) != 1:
                raise KernelError("gla_scan: rows must be contiguous")
        one_row = given and za.shape[0] == 1
        _need(state, torch.float32, "recurrent state")
        _need(out, torch.float32, "recurrence out")
        T = zq.shape[0]
        if not (zq.stride(0) == zk.stride(0) == zv.stride(0)) or zq.shape[1] != heads * dim or \
                zk.shape[1] != heads * dim or zv.shape[1] != heads * vdim or \
                za.shape != (1 if one_row else T, heads * dim) or \
                out.shape != (T, heads * vdim) or state.shape[1:] != (heads, dim, vdim):
            raise KernelError("gla_scan: sizes do not match")
        if bias is not None:
            _need(bias, torch.float32, "decay bias")
        scratch = None
        self._tl_gla_scan_scratch.restype = c_longlong
        n = int(self._tl_gla_scan_scratch(c_int(T), c_int(seq_slot.numel()), c_int(heads), c_int(dim),
                                          c_int(vdim))) if chunked else 0
        if n:
            scratch = (workspace.get("gla_chunks", (n,), torch.float32) if workspace is not None
                       else torch.empty(n, dtype=torch.float32, device=zq.device))
        _check(self._tl_gla_scan(_ptr(zq), _ptr(zk), _ptr(zv), c_int(zq.stride(0)), _ptr(za),
                                 c_int(0 if one_row else za.stride(0)),
                                 _ptr(bias), c_float(tau), c_float(q_scale), _ptr(state), _ptr(out),
                                 c_int(out.stride(0)), _ptr(seq_start), _ptr(seq_slot), c_int(T),
                                 c_int(seq_slot.numel()), c_int(heads), c_int(dim), c_int(vdim), _ptr(scratch),
                                 c_int(1 if given else 0), _stream()), "gla_scan")
        if T > 4 * seq_slot.numel() and not given:
            _check(0, "gla_decay")
        if n:
            _check(0, "gla_chunk_carry")
            _check(0, "gla_chunk_apply")

    # ---- the gated delta rule, short convolutions, and mixers side by side with a factor each ----------
    def delta_prep(self, z: torch.Tensor, taps_w: torch.Tensor, kept: torch.Tensor, y: torch.Tensor,
                   gates: torch.Tensor, neg_a: torch.Tensor, dt_bias: torch.Tensor, col_b: int, col_a: int,
                   token_seq: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor, kv_heads: int,
                   heads: int, dim: int, vdim: int, unit_eps: float, q_scale: float) -> None:
        """From the 32-bit projections `z` (columns q [kv_heads * dim], k [kv_heads * dim], v [heads * vdim],
        then anything; the pre-activations of beta at `col_b` and of the decay at `col_a`, one per head):
        y = [q | k | v] after the causal convolution over `taps_w` [channels, taps] (last column the current
        token's; inputs before the step come from `kept` [slots, taps - 1, channels], oldest first) and silu,
        q and k divided by sqrt(sum of squares + unit_eps), q times `q_scale`;
        gates[t] = [beta (heads) | exp(neg_a * softplus(za + dt_bias)) (heads) | k . q (kv_heads)]."""
        _need(z, torch.float32, "projections", contiguous=False)
        for t, n in ((taps_w, "convolution taps"), (kept, "kept convolution inputs"), (y, "prepared q, k, v"),
                     (gates, "gates"), (neg_a, "decay rate"), (dt_bias, "decay bias")):
            _need(t, torch.float32, n)
        T = z.shape[0]
        channels = 2 * kv_heads * dim + heads * vdim
        taps = taps_w.shape[1]
        if z.stride(1) != 1 or z.shape[1] < max(channels, col_b + heads, col_a + heads) or \
                taps_w.shape != (channels, taps) or kept.shape[1:] != (taps - 1, channels) or \
                y.shape != (T, channels) or gates.shape != (T, 2 * heads + kv_heads) or neg_a.numel() != heads or \
                dt_bias.numel() != heads:
            raise KernelError("delta_prep: sizes do not match")
        _check(self._tl_delta_prep(_ptr(z), c_int(z.stride(0)), _ptr(taps_w), c_int(taps), _ptr(kept), _ptr(y),
                                   c_int(y.stride(0)), _ptr(gates), _ptr(neg_a), _ptr(dt_bias), c_int(col_b),
                                   c_int(col_a), _ptr(token_seq), _ptr(seq_start), _ptr(seq_slot), c_int(T),
                                   c_int(kv_heads), c_int(heads), c_int(dim), c_int(vdim), c_float(unit_eps),
                                   c_float(q_scale), _stream()), "delta_prep")

    def conv_state_update(self, z: torch.Tensor, kept: torch.Tensor, seq_start: torch.Tensor,
                          seq_slot: torch.Tensor, channels: int) -> None:
        """kept[slot] <- the last taps - 1 inputs (the first `channels` columns of `z`) of every sequence of the
        step, older kept inputs moving up where the step brought fewer tokens."""
        _need(z, torch.float32, "projections", contiguous=False)
        _need(kept, torch.float32, "kept convolution inputs")
        if z.stride(1) != 1 or z.shape[1] < channels or kept.shape[2] != channels:
            raise KernelError("conv_state_update: sizes do not match")
        _check(self._tl_conv_state_update(_ptr(z), c_int(z.stride(0)), _ptr(kept), c_int(kept.shape[1] + 1),
                                          _ptr(seq_start), _ptr(seq_slot), c_int(seq_slot.numel()),
                                          c_int(channels), _stream()), "conv_state_update")

    def delta_scan(self, y: torch.Tensor, gates: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                   seq_start: torch.Tensor, seq_slot: torch.Tensor, kv_heads: int, heads: int, dim: int,
                   vdim: int) -> None:
        """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over each sequence's tokens of the step,
        from and into `state` [slots, heads, dim, vdim]; `y` and `gates` as `delta_prep` leaves them."""
        for t, n in ((y, "prepared q, k, v"), (gates, "gates"), (state, "recurrent state"), (out, "recurrence out")):
            _need(t, torch.float32, n)
        T = y.shape[0]
        if y.shape[1] != 2 * kv_heads * dim + heads * vdim or gates.shape != (T, 2 * heads + kv_heads) or \
                out.shape != (T, heads * vdim) or state.shape[1:] != (heads, dim, vdim):
            raise KernelError("delta_scan: sizes do not match")
        _check(self._tl_delta_scan(_ptr(y), c_int(y.stride(0)), _ptr(gates), _ptr(state), _ptr(out),
                                   c_int(out.stride(0)), _ptr(seq_start), _ptr(seq_slot), c_int(T),
                                   c_int(seq_slot.numel()), c_int(kv_heads), c_int(heads), c_int(dim), c_int(vdim),
                                   _stream()), "delta_scan")

    def silu_rows(self, x: torch.Tensor) -> None:
        """x <- silu(x) in place; x 32-bit [T, n], rows may be strided."""
        _need(x, torch.float32, "silu input", contiguous=False)
        if x.stride(1) != 1:
            raise KernelError("silu_rows: rows must be contiguous")
        _check(self._tl_silu_rows(_ptr(x), c_int(x.stride(0)), c_int(x.shape[0]), c_int(x.shape[1]), _stream()),
               "silu_rows")

    def weighted_sum(self, ys, biases, scales, out: torch.Tensor, accumulate: bool) -> None:
        """out (+)= sum_b scales[b] * (ys[b] + biases[b]); biases[b] may be None.  Up to four terms, all
        32-bit [T, n]."""
        n = len(ys)
        _need(out, torch.float32, "weighted sum out")
        for y, b in zip(ys, biases):
            _need(y, torch.float32, "term")
            if y.shape != out.shape:
                raise KernelError("weighted_sum: sizes do not match")
            if b is not None:
                _need(b, torch.float32, "term bias")
                if b.numel() != out.shape[1]:
                    raise KernelError("weighted_sum: a bias has one entry per column")
        yp = (c_void_p * n)(*[y.data_ptr() for y in ys])
        bp = (c_void_p * n)(*[b.data_ptr() if b is not None else None for b in biases])
        sc = (c_float * n)(*[float(s) for s in scales])
        _check(self._tl_weighted_sum(yp, bp, sc, c_int(n), _ptr(out), c_int(out.shape[0]), c_int(out.shape[1]),
                                     c_int(1 if accumulate else 0), _stream()), "weighted_sum")

    # ---- mixture of experts ---------------------------------------------------------------------------
    def moe_route(self, z: torch.Tensor, correction: Optional[torch.Tensor], top: int, idx: torch.Tensor,
                  wt: torch.Tensor) -> None:
        """idx[t, :top] = the router outputs with the largest softmax(z[t]) + correction (ties: the lower
        index), wt = their softmax scores."""
        _need(z, torch.float32, "router logits", contiguous=False)
        _need(idx, torch.int32, "chosen experts")
        _need(wt, torch.float32, "expert weights")
        T, n_out = z.shape
        if z.stride(1) != 1 or idx.shape != (T, top) or wt.shape != (T, top):
            raise KernelError("moe_route: sizes do not match")
        if correction is not None:
            _need(correction, torch.float32, "router correction")
        _check(self._tl_moe_route(_ptr(z), c_int(z.stride(0)), _ptr(correction), c_int(n_out), c_int(top), _ptr(idx),
                                  _ptr(wt), c_int(T), _stream()), "moe_route")

    # ---- rotated queries and keys around the paged attention ----------------------------------------
    def rotary_cache_write(self, z: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, style: int,
                           unit_norm: bool, eps: float, q_out: torch.Tensor, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
                           seq_slot: torch.Tensor, page_table: torch.Tensor, nq: int, nk: int, nv: int, dim: int,
                           vdim: int, slots: int = 1, bias: Optional[torch.Tensor] = None,
                           values_are_keys: bool = False) -> None:
        """The projections `z` (32-bit rows: `nq` query vectors and `nk` key vectors of `dim`, then `nv` value
        heads of `vdim`): the first `rot` entries of every query and key vector are rotated by the token's
        position (`style` 0: pairs (i, i + rot/2), 1: pairs (2i, 2i + 1)), then, with `unit_norm`, the vector
        is divided by its root mean square; q goes to `q_out`, k and v into the pages.  With `slots` > 1 a
        key row of the pages holds `slots` key vectors side by side and query vector j becomes a row of that
        width that is zero outside slot j % slots.  `bias` (32-bit, one number per column of `z`) is added as
        the columns are read.  With `values_are_keys` `z` holds no value columns: a value head is the key
        vector of its head as projected (bias included), before rotation and norm."""
        _need(z, torch.float32, "projections", contiguous=False)
        _need(q_out, self.act_dtype, "q out")
        _need(k_pages, self.act_dtype, "k pages")
        _need(v_pages, self.act_dtype, "v pages")
        _need(page_table, torch.int32, "page table")
        T = z.shape[0]
        cols = (nq + nk) * dim + (0 if values_are_keys else nv * vdim)
        width = slots * dim
        v_col = nq * dim if values_are_keys else (nq + nk) * dim
        if values_are_keys and (vdim != dim or slots != 1):
            raise KernelError("rotary_cache_write: values that are the keys have the keys' size")
        if bias is not None:
            _need(bias, torch.float32, "projection bias")
            if bias.numel() != cols:
                raise KernelError("rotary_cache_write: the bias must have one entry per projected column")
        if z.shape[1] < cols or z.stride(1) != 1 or q_out.shape != (T, nq * width) or nk != nv * slots or \
                k_pages.shape[1:] != (nv, PAGE, width) or v_pages.shape[1:] != (nv, vdim, PAGE):
            raise KernelError("rotary_cache_write: sizes do not match")
        if rot:
            _need(inv_freq, torch.float32, "inverse frequencies")
            if inv_freq.numel() != rot // 2:
                raise KernelError("rotary_cache_write: one inverse frequency per rotated pair is needed")
        _check(self._tl_rotary_cache_write(
            _ptr(z), c_int(z.stride(0)), _ptr(bias), c_int(v_col), _ptr(inv_freq if rot else None), c_int(rot),
            c_int(style),
            c_int(1 if unit_norm else 0), c_float(eps), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(token_pos),
            _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), c_int(T), c_int(nq),
            c_int(nk), c_int(nv), c_int(dim), c_int(vdim), c_int(slots), _stream()), "rotary_cache_write")

    def diff_heads(self, a: torch.Tensor, lam: float, eps: float, mult: float, out: torch.Tensor, heads: int,
                   vdim: int) -> None:
        """a: [T, heads * 2 * vdim] (two maps' outputs per head); out[t, h] = o / rms(o) * mult with
        o = a[t, h, 0] - lam * a[t, h, 1]."""
        _need(a, self.act_dtype, "attention maps")
        _need(out, self.act_dtype, "difference of maps")
        T = a.shape[0]
        if a.shape != (T, heads * 2 * vdim) or out.shape != (T, heads * vdim):
            raise KernelError("diff_heads: sizes do not match")
        _check(self._tl_diff_heads(_ptr(a), c_float(lam), c_float(eps), c_float(mult), _ptr(out), c_int(T),
                                   c_int(heads), c_int(vdim), _stream()), "diff_heads")

    def sigmoid_gate(self, x: torch.Tensor, gate: torch.Tensor) -> None:
        """x *= sigmoid(gate), entry by entry; gate 32-bit, rows may be strided."""
        _need(x, self.act_dtype, "gated tensor")
        _need(gate, torch.float32, "gate", contiguous=False)
        if gate.shape != x.shape or gate.stride(1) != 1:
            raise KernelError("sigmoid_gate: sizes do not match")
        _check(self._tl_sigmoid_gate(_ptr(x), _ptr(gate), c_int(gate.stride(0)), c_int(x.shape[0]),
                                     c_int(x.shape[1]), _stream()), "sigmoid_gate")

    # ---- a block with a norm before and after each sublayer ------------------------------------------
    def norm_add_norm(self, y: torch.Tensor, w_out: torch.Tensor, eps_out: float, x: torch.Tensor,
                      w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0,
                      xn: Optional[torch.Tensor] = None) -> None:
        """x += y / rms(y) * w_out (32-bit stream, in place); with `w_next`, also xn = x / rms(x) * w_next in
        the activation type."""
        _need(y, torch.float32, "sublayer output", contiguous=False)
        _need(x, torch.float32, "stream")
        T, H = x.shape
        if y.shape != (T, H) or y.stride(1) != 1 or w_out.numel() != H:
            raise KernelError("norm_add_norm: sizes do not match")
        w32 = w_out.dtype == torch.float32
        if not w32 and w_out.dtype != torch.bfloat16:
            raise KernelError("norm_add_norm: norm weights must be 32-bit or bfloat16")
        if w_next is not None:
            if w_next.dtype != w_out.dtype or w_next.numel() != H or xn is None:
                raise KernelError("norm_add_norm: the next norm must match the first")
            _need(xn, self.act_dtype, "normed stream")
            if xn.shape != (T, H):
                raise KernelError("norm_add_norm: sizes do not match")
        _check(self._tl_norm_add_norm(_ptr(y), c_int(y.stride(0)), _ptr(w_out), _ptr(w_next), c_int(1 if w32 else 0),
                                      c_float(eps_out), c_float(eps_next), _ptr(x), _ptr(xn), c_int(T), c_int(H),
                                      _stream()), "norm_add_norm")

    def relu_squared(self, z: torch.Tensor, out: torch.Tensor) -> None:
        """out = max(z, 0)^2; z 32-bit, rows may be strided."""
        _need(z, torch.float32, "pre-activations", contiguous=False)
        _need(out, self.act_dtype, "activations")
        if z.shape != out.shape or z.stride(1) != 1:
            raise KernelError("relu_squared: sizes do not match")
        _check(self._tl_relu_squared(_ptr(z), c_int(z.stride(0)), _ptr(out), c_int(out.shape[0]), c_int(out.shape[1]),
                                     _stream()), "relu_squared")

    def clamped_glu(self, z: torch.Tensor, limit: float, alpha: float, out: torch.Tensor) -> None:
        """z: [T, 2 n] 32-bit, gate columns then up columns: g = min(g, limit), u = clamp(u, -limit, limit),
        out = g * sigmoid(alpha g) * (u + 1)."""
        _need(z, torch.float32, "pre-activations", contiguous=False)
        _need(out, self.act_dtype, "activations")
        T, n = out.shape
        if z.shape != (T, 2 * n) or z.stride(1) != 1:
            raise KernelError("clamped_glu: sizes do not match")
        _check(self._tl_clamped_glu(_ptr(z), c_int(z.stride(0)), c_float(limit), c_float(alpha), _ptr(out), c_int(T),
                                    c_int(n), _stream()), "clamped_glu")

    def moe_route_grouped(self, z: torch.Tensor, groups: int, keep: int, top: int, scale: float, idx: torch.Tensor,
                          wt: torch.Tensor) -> None:
        """s = sigmoid(z[t]); only experts of the `keep` groups (of `groups` equal groups of neighbours) with
        the largest sum of their two best s can be chosen; idx[t, :top] = the largest s among them (ties: the
        lower index), wt = their s / (their sum + 1e-20) * scale."""
        _need(z, torch.float32, "router logits", contiguous=False)
        _need(idx, torch.int32, "chosen experts")
        _need(wt, torch.float32, "expert weights")
        T, n_out = z.shape
        if z.stride(1) != 1 or idx.shape != (T, top) or wt.shape != (T, top):
            raise KernelError("moe_route_grouped: sizes do not match")
        _check(self._tl_moe_route_grouped(_ptr(z), c_int(z.stride(0)), c_int(n_out), c_int(groups), c_int(keep),
                                          c_int(top), c_float(scale), _ptr(idx), _ptr(wt), c_int(T), _stream()),
               "moe_route_grouped")

    def moe_plan(self, idx: torch.Tensor, experts: int, offsets: torch.Tensor, row_token: torch.Tensor,
                 row_of: torch.Tensor) -> None:
        """Groups the (token, choice) pairs by expert: offsets [experts + 1], row_token [pairs], row_of
        [tokens, top] (-1 where the chosen expert has no matrices)."""
        for t, n in ((idx, "chosen experts"), (offsets, "offsets"), (row_token, "row tokens"), (row_of, "rows")):
            _need(t, torch.int32, n)
        T, top = idx.shape
        if offsets.numel() != experts + 1 or row_token.numel() < T * top or row_of.shape != idx.shape:
            raise KernelError("moe_plan: sizes do not match")
        _check(self._tl_moe_plan(_ptr(idx), c_int(T * top), c_int(top), c_int(experts), _ptr(offsets),
                                 _ptr(row_token), _ptr(row_of), _stream()), "moe_plan")

    def moe_gemm(self, a: torch.Tensor, row_token: Optional[torch.Tensor], w: torch.Tensor, c: torch.Tensor,
                 offsets: torch.Tensor, up: bool, limit: float = 0.0, alpha: float = 0.0) -> None:
        """The experts' products over rows grouped by expert.  up: c[row] = act(gate, up) of a[row_token[row]]
        with w [experts, 2 N, K]; else c[row] (32-bit) = a[row] . w[expert] with w [experts, N, K]."""
        _need(a, self.act_dtype, "expert input")
        _need(w, self.act_dtype, "expert matrices")
        _need(c, self.act_dtype if up else torch.float32, "expert output")
        E, rows_w, K = w.shape
        N = rows_w // 2 if up else rows_w
        if a.shape[1] != K or c.shape[1] != N or offsets.numel() != E + 1 or (up and row_token is None):
            raise KernelError("moe_gemm: sizes do not match")
        if self.act_dtype == torch.bfloat16:
            # the tensor-core kernel, where alignments allow it
            self.lib.tl_moe_gemm_mma.restype = c_int
            st = self.lib.tl_moe_gemm_mma(_ptr(a), c_int(a.stride(0)), _ptr(row_token), _ptr(w), _ptr(c),
                                          c_int(c.stride(0)), _ptr(offsets), c_int(E), c_int(c.shape[0]), c_int(N),
                                          c_int(K), c_int(1 if up else 0), c_float(limit), c_float(alpha), _stream())
            if st != -2:
                _check(st, "moe_gemm_mma")
                return
        _check(self._tl_moe_gemm(_ptr(a), c_int(a.stride(0)), _ptr(row_token), _ptr(w), _ptr(c), c_int(c.stride(0)),
                                 _ptr(offsets), c_int(E), c_int(c.shape[0]), c_int(N), c_int(K), c_int(1 if up else 0),
                                 c_float(limit), c_float(alpha), _stream()), "moe_gemm")

    def moe_combine(self, yk: torch.Tensor, row_of: torch.Tensor, wt: torch.Tensor, h: torch.Tensor,
                    out: torch.Tensor, accumulate: bool) -> None:
        """out[t] (+)= sum_k wt[t, k] * (yk[row_of[t, k]] if row_of[t, k] >= 0 else h[t])."""
        _need(yk, torch.float32, "expert outputs")
        _need(row_of, torch.int32, "rows")
        _need(wt, torch.float32, "expert weights")
        _need(h, self.act_dtype, "feed-forward input")
        _need(out, torch.float32, "feed-forward output", contiguous=False)
        T, top = row_of.shape
        H = h.shape[1]
        if out.shape != (T, H) or yk.shape[1] != H or wt.shape != row_of.shape or out.stride(1) != 1:
            raise KernelError("moe_combine: sizes do not match")
        _check(self._tl_moe_combine(_ptr(yk), _ptr(row_of), _ptr(wt), _ptr(h), _ptr(out), c_int(out.stride(0)),
                                    c_int(T), c_int(H), c_int(top), c_int(1 if accumulate else 0), _stream()),
               "moe_combine")


class SamplingOps:
    def __init__(self):
        self.lib = build.load_library("sampling")
        self.lib.tl_argmax.restype = c_int
        self.lib.tl_sample.restype = c_int

    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        _need(logits, torch.float32, "argmax logits", contiguous=False)
        _need(out, torch.int32, "argmax out")
        rows, V = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("argmax: the last dimension must be contiguous")
        _check(self.lib.tl_argmax(_ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(V),
                                  _ptr(out), _stream()), "argmax")

    def sample(self, logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
               uniform: torch.Tensor, out: torch.Tensor) -> None:
        _need(logits, torch.float32, "sample logits", contiguous=False)
        _need(uniform, torch.float32, "sample uniform")
        _need(out, torch.int32, "sample out")
        rows, V = logits.shape
        if logits.stride(1) != 1 or uniform.numel() < rows or out.numel() < rows:
            raise KernelError("sample: bad arguments")
        _check(self.lib.tl_sample(_ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(V),
                                  c_float(temperature), c_int(top_k), c_float(top_p),
                                  _ptr(uniform), _ptr(out), _stream()), "sample")


_core: dict = {}
_sampling: list = []


def core_ops(act_dtype: torch.dtype) -> CoreOps:
    if act_dtype not in _core:
        _core[act_dtype] = CoreOps(act_dtype)
    return _core[act_dtype]


def sampling_ops() -> SamplingOps:
    if not _sampling:
        _sampling.append(SamplingOps())
    return _sampling[0]
