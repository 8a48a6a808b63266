"""Typed Python faces of the ``extern "C"`` kernel launchers.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, shapes), passes raw pointers and the current CUDA stream, and
turns a refusal or a launch error into an exception.  Nothing here computes
on the host and nothing falls back to another implementation.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import guard
from .csrc.build import load_library
from .errors import ExtensionMissing, KernelError, Unsupported

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; the same constant as LLMX_PAGE in common.cuh
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}

_REFUSALS = {
    1: "a size or stride is out of range",
    2: "unsupported combination of dtypes",
    3: "a size exceeds what this kernel's shared memory or grid allows",
    4: "a required table is missing",
}


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise ExtensionMissing("no CUDA device is available; llmoxide_b200 has no CPU path")


def _tag(t: torch.Tensor) -> int:
    try:
        return _DTYPE_TAG[t.dtype]
    except KeyError:
        raise Unsupported(f"dtype {t.dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _ptr(t):
    """A tensor's address as the plain integer (None for no tensor) that a c_void_p argument converts itself."""
    return None if t is None else t.data_ptr()


# The current stream's handle without building a torch.cuda.Stream object for every launch (a prompt step of a
# few tokens launches some 300 kernels and is bound by the host).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


launch_count = 0  # kernels of this package launched (or replayed from a graph) so far


def _check(code: int, what: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise Unsupported(f"{what}: refused, {_REFUSALS.get(-code, f'code {-code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("a kernel was handed a tensor that is not on the GPU")


def _contig(name, t):
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_fn_cache: dict = {}
_libs_ready: set = set()
_overlap = True


def _library(lib_name: str):
    """The library, loaded onto the GPU while nothing else runs there.  Rule: no CUDA module is loaded in the
    middle of a step, because loading one synchronises with the device while hundreds of launches that overlap
    one another may still be pending.  So the first use of a library waits for the GPU to drain and makes the
    module resident (``llmx_touch``) before anything of it is launched; an engine names its libraries when it
    is built (``preload``), so that no step has to."""
    global launch_count
    lib = load_library(lib_name)
    if lib_name not in _libs_ready:
        if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            torch.cuda.synchronize()
            touch = getattr(lib, "llmx_touch", None)
            if touch is not None:
                touch.restype = c_int
                _check(touch(), f"loading {lib_name}")
                launch_count -= 1
            torch.cuda.synchronize()
            if lib_name in _STATUS_SLOTS and hasattr(lib, "llmx_set_status_word"):
                lib.llmx_set_status_word.argtypes = [c_void_p]
                lib.llmx_set_status_word.restype = c_int
                _check(lib.llmx_set_status_word(c_void_p(status_word(lib_name).data_ptr())),
                       f"registering the status word of {lib_name}")
                launch_count -= 1
            _libs_ready.add(lib_name)
        if hasattr(lib, "llmx_set_pdl"):
            lib.llmx_set_pdl(int(_overlap))
    return lib


# ---- failure reports -------------------------------------------------------
# One word per library in page-locked host memory that its kernels can write: a bounded wait that ran out,
# or a request a kernel could not serve, leaves a code there.  The host looks at the words whenever it has
# waited for a step anyway (no copy, no extra synchronisation).

_STATUS_SLOTS = {"gemm_tc": 0, "attention_prefill_tc": 1, "attention_decode": 2, "sampling": 3, "moe_tc": 4,
                 "short_conv": 5, "stream_mix": 6, "moe": 7, "attention": 8, "latent_attention": 9}
_STATUS_MEANING = {
    "gemm_tc": {1: "the producer's wait for a free stage ran out", 2: "the MMA issuer's wait for a stage's data ran out",
                3: "the epilogue's wait for an accumulator ran out", 4: "the MMA issuer's wait for a drained accumulator ran out",
                11: "CTA pair: the producer's wait for a free stage ran out", 12: "CTA pair: the MMA issuer's wait for a stage's data ran out",
                13: "CTA pair: the epilogue's wait for an accumulator ran out",
                14: "CTA pair: the MMA issuer's wait for a drained accumulator ran out"},
    "attention_prefill_tc": {20: "its shared memory is not 1024-byte aligned"},
    "moe_tc": {1: "the producer's wait for a free stage ran out", 2: "the MMA issuer's wait for a stage's data ran out",
               3: "the epilogue's wait for an accumulator ran out", 4: "the MMA issuer's wait for a drained accumulator ran out"},
    "attention_decode": {1: "a copy into shared memory never completed", 2: "its shared memory is not 1024-byte aligned"},
    "sampling": {1: "top_p < 1 over more candidates than the kernel sorts", 2: "top_k beyond what the kernel sorts"},
    "short_conv": {1: "a token's sequence, position, slot or page lies outside the launch's arrays",
                   2: "a sequence's rows or slot lie outside the launch's arrays (state update)"},
    "stream_mix": {1: "a wanted row lies outside the stream"},
    "moe": {1: "a token's router scores hold a NaN (no expert compares greater than none)",
            2: "an expert id outside the router's experts reached the sort",
            3: "a token id outside the routing table, or a table entry that names no expert"},
    "attention": {1: "a block's row has no page in the store of one row per block",
                  2: "a block's positions are no longer held by the cache"},
    "latent_attention": {1: "a token's sequence, position or page lies outside the launch's arrays"},
}
_status_host = None


def status_words() -> torch.Tensor:
    """The page-locked int32 words, one per library that reports (see ``_STATUS_SLOTS``)."""
    global _status_host
    if _status_host is None:
        _status_host = torch.zeros(16, dtype=torch.int32).pin_memory()
    return _status_host


def status_word(lib_name: str) -> torch.Tensor:
    i = _STATUS_SLOTS[lib_name]
    return status_words()[i : i + 1]


def check_status() -> None:
    """Raises ``KernelError`` if a kernel has left a report since the last call, and clears it.  Meaningful
    once the host has waited for the work in question (the words are written as the failure happens)."""
    if _status_host is None:
        return
    words = _status_host.numpy()
    if not words.any():
        return
    found = []
    for name, i in _STATUS_SLOTS.items():
        code = int(words[i])
        if code:
            what = _STATUS_MEANING.get(name, {}).get(code, "a bounded wait ran out")
            found.append(f"{name}: {what} (code {code})")
    words[:] = 0
    raise KernelError("a kernel reported a failure; the step's results are not to be used: " + "; ".join(found))


def test_waits(lib_name: str, cycles: int = 0, withhold: bool = False) -> None:
    """For tests of the failure path: the limit of the library's bounded waits in clock cycles (0: the default
    of about two seconds) and whether one role leaves out one arrival, so that a wait runs out, is reported
    and the kernel winds down through its normal exit."""
    f = _fn(lib_name, "llmx_test_waits", [c_longlong, c_int])
    torch.cuda.synchronize()
    code = f(int(cycles), int(withhold))
    if code:
        raise KernelError(f"{lib_name}: CUDA error {code} setting the wait limit")


def set_overlap(on: bool) -> None:
    """Whether the kernels launched from now on may start while the kernel before them still runs
    (programmatic stream serialization; every kernel waits for its inputs itself).  On for decode steps,
    which are chains of short kernels; the engine switches it off for prompt steps."""
    global _overlap
    if on == _overlap:
        return
    _overlap = on
    for name in _libs_ready:
        lib = load_library(name)
        if hasattr(lib, "llmx_set_pdl"):
            lib.llmx_set_pdl(int(on))


def _fn(lib_name: str, fn_name: str, argtypes):
    key = (lib_name, fn_name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(_library(lib_name), fn_name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


def preload(lib_names) -> None:
    """Makes the named libraries resident now (an engine does this when it is built, so that no step has to)."""
    for name in lib_names:
        _library(name)


# ---------------------------------------------------------------------------


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t,:] = float32(table[tokens[t],:]) * scale.  tokens int32 [T]; out float32 [T,d]."""
    _dev(table, tokens, out)
    _contig("table", table), _contig("out", out)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32
    f = _fn("elementwise", "llmx_embed",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(table), _tag(table), _ptr(tokens), _ptr(out), tokens.numel(), table.shape[1],
             table.shape[0], scale, _stream()), "embed")


def embed_positions(table, positions, tokens, token_pos, h, scale: float = 1.0) -> None:
    """h[s][t,:] = float32(table[tokens[t],:]) * scale + float32(positions[token_pos[t],:]) for every copy s of the
    residual stream; h float32 [T,d] or [S,T,d]; ``positions`` None or a table of the same dtype and width."""
    _dev(table, positions, tokens, token_pos, h)
    _contig("table", table), _contig("h", h)
    assert tokens.dtype == torch.int32 and h.dtype == torch.float32
    if positions is not None:
        _contig("positions", positions)
        assert positions.dtype == table.dtype and positions.shape[1] == table.shape[1] and token_pos.dtype == torch.int32
    n_streams, stride = (h.shape[0], h.stride(0)) if h.dim() == 3 else (1, 0)
    f = _fn("elementwise", "llmx_embed_pos",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
             c_void_p])
    _check(f(_ptr(table), _ptr(positions), _tag(table), _ptr(tokens), _ptr(token_pos), _ptr(h), stride, n_streams,
             tokens.numel(), table.shape[1], table.shape[0], 0 if positions is None else positions.shape[0], scale,
             _stream()), "embed_positions")


def stream_mix_norm(h, delta, mix, write, read, gain, eps: float, out, rows=None, write_h: bool = True) -> None:
    """Copies of the residual stream h float32 [S,T,d].  First the update a sublayer owes, when ``mix`` is given:
    h_r <- sum_s mix[s,r] h_s + write[r] * delta (``delta`` None, [T,d] or split partials [P,T,d] added in order;
    the copies are stored when ``write_h``).  Then out[r] = rmsnorm(sum_s read[s] h_s)[rows[r]] * gain (``read``
    None: the plain sum; ``out`` None: only the update)."""
    _dev(h, delta, mix, write, read, gain, out, rows)
    _contig("h", h)
    assert h.dtype == torch.float32 and h.dim() == 3
    S, T, d = h.shape
    n_split, stride, dtag = 1, 0, F32
    if delta is not None:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == (T, d), (delta.shape, h.shape)
        n_split, stride, dtag = delta.shape[0], delta.stride(0), _tag(delta)
    for w, n in ((mix, S * S), (write, S), (read, S)):
        assert w is None or (w.dtype == torch.float32 and w.numel() == n and w.is_contiguous())
    n_rows = T if rows is None else rows.numel()
    if out is not None:
        _contig("out", out)
        assert out.shape[0] >= n_rows and out.shape[-1] == d and gain.dtype == torch.float32
    f = _fn("stream_mix", "llmx_stream_mix_norm",
            [c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), h.stride(0), S, _ptr(delta), dtag, n_split, stride, _ptr(mix), _ptr(write), _ptr(read), _ptr(rows),
             n_rows, _ptr(gain), eps, _ptr(out), _tag(out) if out is not None else F32, d, int(write_h), T, _stream()),
           "stream_mix_norm")


def conv_rope_cache(proj, state, conv_w, taps: int, q_out, k_cache, v_cache, block_table, ctx, cos, sin, n_rot: int,
                    v_first, v_lambda, v_mix_mode: int, n_heads: int, n_kv_heads: int, head_dim: int,
                    v_head_dim: int, inline_state: bool = False) -> None:
    """A short causal convolution (``conv_w`` float32 [taps, C], tap-major; taps 0: none) over the fused q|k|v projection
    ``proj`` ([T,C] or float32 partials [P,T,C]) with the sequences' earlier rows from ``state`` float32
    [slots, taps-1, C]; then q and k rotated (q to ``q_out`` [T,H*D], k to the cache) and v written to the cache:
    as it is (``v_mix_mode`` 0), also copied to ``v_first`` float32 [T,G*Dv] (1), or mixed with it as
    (1 - l) v + l v_first, l = ``v_lambda[0]`` (2).  ``ctx``: the step's index arrays.  ``inline_state``: every
    sequence brings exactly one token, and the kernel moves the state on itself (no ``conv_state_update`` then)."""
    _dev(proj, state, conv_w, q_out, k_cache, v_cache, block_table, cos, sin, v_first, v_lambda)
    _contig("proj", proj), _contig("q_out", q_out), _contig("block_table", block_table)
    n_split, stride = (proj.shape[0], proj.stride(0)) if proj.dim() == 3 else (1, 0)
    T = proj.shape[-2]
    C = (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_head_dim
    assert proj.shape[-1] == C and q_out.shape == (T, n_heads * head_dim)
    assert k_cache.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    if taps:
        assert conv_w.dtype == torch.float32 and conv_w.shape == (taps, C) and conv_w.is_contiguous()
    if taps > 1:
        assert state.dtype == torch.float32 and state.shape[1:] == (taps - 1, C) and state.is_contiguous()
    if v_mix_mode:
        assert v_first.dtype == torch.float32 and v_first.shape == (T, n_kv_heads * v_head_dim) and v_first.is_contiguous()
    f = _fn("short_conv", "llmx_conv_rope_cache",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p])
    _check(f(_ptr(proj), _tag(proj), n_split, stride, _ptr(state), int(bool(inline_state) and taps > 1), _ptr(conv_w), taps, _ptr(q_out), _tag(q_out),
             _ptr(k_cache), _ptr(v_cache), _tag(k_cache), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
             _ptr(ctx.token_pos), _ptr(ctx.seq_start), _ptr(ctx.seq_past), _ptr(ctx.seq_slot), _ptr(cos), _ptr(sin), n_rot,
             _ptr(v_first), _ptr(v_lambda), v_mix_mode, T, n_heads, n_kv_heads, head_dim, v_head_dim, ctx.n_seqs,
             state.shape[0] if state is not None else 1 << 30, k_cache.shape[0], _stream()), "conv_rope_cache")


def conv_state_update(proj, state, taps: int, ctx) -> None:
    """Moves the convolution's state on by the step's tokens: afterwards ``state[slot]`` holds the projected rows
    of every sequence's last taps-1 positions."""
    if taps <= 1:
        return
    _dev(proj, state)
    n_split, stride = (proj.shape[0], proj.stride(0)) if proj.dim() == 3 else (1, 0)
    C = proj.shape[-1]
    assert state.dtype == torch.float32 and state.shape[1:] == (taps - 1, C) and state.is_contiguous()
    f = _fn("short_conv", "llmx_conv_state_update",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), _tag(proj), n_split, stride, _ptr(state), taps, _ptr(ctx.seq_start), _ptr(ctx.seq_slot),
             ctx.n_seqs, C, proj.shape[-2], state.shape[0], _stream()), "conv_state_update")


CONV_MAX_TAPS = 16     # the same constant as SC_MAX_TAPS in short_conv.cu


def residual_conv(x, state, conv_w, taps: int, out, ctx, inline_state: bool = False) -> None:
    """out = x + conv(x): a causal convolution over time on every channel, y_p = sum_j w[j] x_(p - taps + 1 + j),
    zeros before a sequence's start.  x, out [T, C] of one dtype; ``conv_w`` float32 [taps, C]; ``state`` float32
    [slots, taps-1, C], the last taps-1 rows of x of every sequence (read here; moved on here as well when
    ``inline_state`` and every sequence brings one token, else by ``conv_state_update``)."""
    _dev(x, state, conv_w, out)
    _contig("x", x), _contig("out", out), _contig("conv_w", conv_w)
    C = x.shape[1]
    assert out.shape == x.shape and out.dtype == x.dtype and conv_w.dtype == torch.float32 and conv_w.shape == (taps, C)
    assert taps == 1 or (state is not None and state.dtype == torch.float32 and state.shape[1:] == (taps - 1, C)
                         and state.is_contiguous())
    f = _fn("short_conv", "llmx_residual_conv",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_longlong, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _tag(x), _ptr(state), int(inline_state), _ptr(conv_w), taps, _ptr(out), _ptr(ctx.token_seq),
             _ptr(ctx.token_pos), _ptr(ctx.seq_start), _ptr(ctx.seq_past), _ptr(ctx.seq_slot), x.shape[0], C, ctx.n_seqs,
             state.shape[0] if state is not None else 0, _stream()), "residual_conv")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place; x float32, contiguous."""
    _dev(x)
    _contig("x", x)
    assert x.dtype == torch.float32 and cap > 0
    f = _fn("elementwise", "llmx_softcap", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), x.numel(), cap, _stream()), "softcap")


def scale_(x: torch.Tensor, factor: float) -> None:
    """x *= factor in place; x float32, contiguous."""
    _dev(x)
    _contig("x", x)
    assert x.dtype == torch.float32
    f = _fn("elementwise", "llmx_scale", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), x.numel(), factor, _stream()), "scale")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t, :] += bias in place (float32 sum); y [T, d] float32 or bfloat16, bias float32 [d]."""
    _dev(y, bias)
    _contig("y", y)
    assert y.dim() == 2 and bias.dtype == torch.float32 and bias.numel() == y.shape[1] and bias.is_contiguous()
    f = _fn("post_norm", "llmx_add_bias", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(y), _tag(y), y.shape[0], y.shape[1], _ptr(bias), _stream()), "add_bias")


def add_rms_norm(h: torch.Tensor, delta, gain: torch.Tensor, eps: float, out, rows=None,
                 write_h: bool = True) -> None:
    """h float32 [T,d] is the residual stream.  ``delta`` is None or [S,T,d]
    (split partials, summed in order).  v = h + sum(delta); h = v when
    ``write_h``; out[r] = rmsnorm(v[rows[r]]) * gain, or for every row without
    ``rows``.  ``out`` may be None when only the sum is wanted."""
    _dev(h, delta, gain, out, rows)
    assert h.dtype == torch.float32 and gain.dtype == torch.float32
    _contig("h", h)
    d = h.shape[-1]
    n_split, stride, dtag = 1, 0, F32
    if delta is not None:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == h.shape, (delta.shape, h.shape)
        n_split, stride, dtag = delta.shape[0], delta.stride(0), _tag(delta)
    n_rows = h.shape[0] if rows is None else rows.numel()
    if out is not None:
        _contig("out", out)
        assert out.shape[0] >= n_rows and out.shape[-1] == d
    f = _fn("elementwise", "llmx_add_rms_norm",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_float, c_void_p,
             c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(delta), dtag, n_split, stride, _ptr(rows), n_rows, _ptr(gain), eps, _ptr(out),
             _tag(out) if out is not None else F32, d, int(write_h), _stream()), "add_rms_norm")


def post_norm_add_norm(h, groups, bias, post_gain, post_center: bool, post_eps: float, gain, center: bool, eps: float,
                       out, rows=None, write_h: bool = True, gate=None) -> None:
    """A sublayer's result normed before it joins the residual stream ``h`` (float32 [T, d], in place), and the norm
    the next sublayer reads.  ``groups``: up to two (delta, weight), delta [T, d] or split partials [S, T, d] summed
    in order; y = sum_g weight_g * delta_g + ``bias``; with ``post_gain`` y = norm(y) * post_gain; v = h + y (stored
    when ``write_h``); with ``out`` out[r] = norm(v[rows[r]]) * gain (every row without ``rows``).  A norm with
    ``center`` subtracts the mean (layer norm without bias), without it is an RMS norm; both are float32.
    ``gate`` = (z, b): y is multiplied by sigmoid(z + b) element by element before its norm; z [T, d] or split
    partials [S, T, d], b float32 [d] or None."""
    deltas = [g[0] for g in groups]
    _dev(h, bias, post_gain, gain, out, rows, *deltas)
    assert h.dtype == torch.float32 and h.dim() == 2 and len(groups) <= 2
    _contig("h", h)
    d = h.shape[1]
    args = []
    for delta, weight in groups:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == h.shape, (delta.shape, h.shape)
        args += [_ptr(delta), _tag(delta), delta.shape[0], delta.stride(0), float(weight)]
    args += [None, F32, 1, 0, 1.0] * (2 - len(groups))
    for v in (bias, post_gain, gain):
        assert v is None or (v.dtype == torch.float32 and v.numel() == d and v.is_contiguous())
    n_rows = h.shape[0] if rows is None else rows.numel()
    if out is not None:
        _contig("out", out)
        assert out.shape[0] >= n_rows and out.shape[-1] == d
    gate_args = [None, F32, 1, 0, None]
    if gate is not None:
        z, zb = gate
        _dev(z, zb)
        _contig("gate", z)
        assert groups, "a gate multiplies a result"
        if z.dim() == 2:
            z = z.unsqueeze(0)
        assert z.shape[1:] == h.shape and (zb is None or (zb.dtype == torch.float32 and zb.numel() == d
                                                          and zb.is_contiguous()))
        gate_args = [_ptr(z), _tag(z), z.shape[0], z.stride(0), _ptr(zb)]
    f = _fn("post_norm", "llmx_post_norm_add_norm_gated",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_float, c_void_p, c_int, c_int, c_longlong, c_float, c_void_p,
             c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int,
             c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(_ptr(h), *args, _ptr(bias), _ptr(post_gain), int(post_center), post_eps, _ptr(rows), n_rows, _ptr(gain),
             int(center), eps, _ptr(out), _tag(out) if out is not None else F32, d, int(write_h), *gate_args, _stream()),
           "post_norm_add_norm")


ADD_SLICE = 512  # columns per CTA of add_gain_sumsq; the same constant as in elementwise.cu


def add_gain_sumsq(h: torch.Tensor, delta, gain: torch.Tensor, x_out: torch.Tensor, sumsq: torch.Tensor) -> None:
    """The residual add and the first half of an RMSNorm for a step of few tokens: h float32 [T,d] += delta
    (None, [T,d] or split partials [S,T,d], added in order); x_out = bfloat16(h * gain); sumsq[s, t] = the sum
    of squares of h[t] over the s-th slice of ``ADD_SLICE`` columns.  The matrix product that reads ``x_out``
    applies the scale (``gemm_tc(scale=...)``)."""
    _dev(h, delta, gain, x_out, sumsq)
    _contig("h", h), _contig("x_out", x_out)
    T, d = h.shape
    assert h.dtype == torch.float32 and gain.dtype == torch.float32 and gain.shape == (d,)
    assert x_out.shape == (T, d) and x_out.dtype == torch.bfloat16 and d % 4 == 0
    n_slices = (d + ADD_SLICE - 1) // ADD_SLICE
    assert sumsq.dtype == torch.float32 and sumsq.shape[0] >= n_slices and sumsq.stride(0) >= T and sumsq.stride(1) == 1
    n_split, stride, dtag = 1, 0, F32
    if delta is not None:
        _contig("delta", delta)
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        assert delta.shape[1:] == h.shape
        n_split, stride, dtag = delta.shape[0], delta.stride(0), _tag(delta)
    f = _fn("elementwise", "llmx_add_gain_sumsq",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(delta), dtag, n_split, stride, _ptr(gain), _ptr(x_out), _ptr(sumsq), sumsq.stride(0), T, d,
             _stream()), "add_gain_sumsq")


def qk_norm_rope_cache(qkv, q_out, k_cache, v_cache, block_table, token_seq, token_pos, q_gain, k_gain,
                       eps: float, cos, sin, n_rot: int, n_heads: int, n_kv_heads: int, head_dim: int,
                       write_cache: bool = True, v_head_dim=None, bias=None) -> None:
    """``bias`` float32, as long as a row of qkv: the projection's bias, added first.
    qkv [T,(H+2G)*D], or float32 split partials [S,T,(H+2G)*D] summed in
    order -> q_out [T,H*D] (normed, rotated) and, when ``write_cache``, k
    (normed, rotated) and v into the paged cache entry ``k_cache``/``v_cache``
    [n_pages,G,PAGE,D] at each token's position."""
    _dev(qkv, q_out, k_cache, v_cache, block_table, token_seq, token_pos)
    _contig("qkv", qkv), _contig("q_out", q_out), _contig("block_table", block_table)
    n_split, stride = 1, 0
    if qkv.dim() == 3:
        n_split, stride = qkv.shape[0], qkv.stride(0)
    T = qkv.shape[-2]
    v_head_dim = v_head_dim or head_dim          # values may have a size of their own (the row's last part)
    assert qkv.shape[-1] == (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_head_dim
    assert q_out.shape[-1] == n_heads * head_dim
    assert k_cache.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    if head_dim > 256 or head_dim % 2:
        raise Unsupported(f"head_dim {head_dim}: the q/k norm and rotation kernel takes even sizes up to 256")
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == qkv.shape[-1] and bias.is_contiguous()
                            and bias.is_cuda)
    f = _fn("elementwise", "llmx_qk_norm_rope_cache_biased",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(qkv), _tag(qkv), n_split, stride, _ptr(q_out), _tag(q_out), _ptr(k_cache), _ptr(v_cache),
             _tag(k_cache), _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(token_pos),
             _ptr(q_gain), _ptr(k_gain), eps, _ptr(cos), _ptr(sin), n_rot, T, n_heads, n_kv_heads, head_dim,
             v_head_dim, int(write_cache), _ptr(bias), _stream()), "qk_norm_rope_cache")


GATE_ACTS = {"silu": 0, "relu": 1, "clamped_swish": 2, "gelu_tanh": 3}


def gate_act_args(activation="silu") -> tuple:
    """(kind, slope, limit, shift) as the kernels take them.  ``activation``: "silu", "relu", or
    ("clamped_swish", slope, limit, shift): min(g, limit) * sigmoid(slope * min(g, limit)) * (clamp(u, +-limit) + shift)."""
    if isinstance(activation, str):
        return GATE_ACTS[activation], 1.0, 0.0, 0.0
    name, slope, limit, shift = activation
    return GATE_ACTS[name], float(slope), float(limit), float(shift)


def silu_gate(gu: torch.Tensor, out: torch.Tensor, block: int = 0, activation="silu", bias=None) -> None:
    """gu [S,T,2F] or [T,2F] -> out [T,F] = act(gate) * up (SiLU unless ``activation`` says otherwise, see
    ``gate_act_args``).  ``block`` = 0: gate columns, then up columns; ``block`` > 0: blocks of that many gate
    columns each followed by the up columns of the same features."""
    _dev(gu, out)
    _contig("gu", gu), _contig("out", out)
    if gu.dim() == 2:
        gu = gu.unsqueeze(0)
    S, T, F2 = gu.shape
    assert out.shape == (T, F2 // 2)
    # ``bias`` float32 [2F]: the projection's bias in the order of gu's columns, added before the activation
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == F2 and bias.is_contiguous() and bias.is_cuda)
    f = _fn("elementwise", "llmx_gate_act_biased",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float,
             c_void_p, c_void_p])
    _check(f(_ptr(gu), _tag(gu), S, gu.stride(0), _ptr(out), _tag(out), T, F2 // 2, block, *gate_act_args(activation),
             _ptr(bias), _stream()), "gate_act")


def sum_splits(parts: torch.Tensor, out: torch.Tensor) -> None:
    """out = parts.sum(0) with the partials added in order; parts [S, ...]."""
    _dev(parts, out)
    _contig("parts", parts), _contig("out", out)
    assert parts.shape[1:] == out.shape
    f = _fn("elementwise", "llmx_sum_splits",
            [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(parts), _tag(parts), parts.shape[0], parts.stride(0), _ptr(out), _tag(out), out.numel(),
             _stream()), "sum_splits")


def attention_paged(q, out, k_cache, v_cache, block_table, token_seq, token_pos, n_heads: int,
                    n_kv_heads: int, head_dim: int, window, scale: float, v_head_dim=None, keep_first: int = 0,
                    sink: float = 0.0, chunk: int = 0, pool: int = 0, pool_k=None, pool_v=None, pool_table=None,
                    gate=None) -> None:
    """General attention over the paged cache; q [T,H*D] (rows may be the first columns of wider rows), out
    [T,H*Dv].  Under a window the first ``keep_first`` keys of a sequence stay visible.  ``sink`` is added to the
    softmax's denominator (as many keys of score 0 that have no value).  With ``chunk`` n > 0 a query sees only the
    keys of its own chunk of n positions, counted from the sequence's position 0.  With ``pool`` n > 0 (beside a
    window) every block of n positions that lies wholly before the window is seen as row b of ``pool_k`` / ``pool_v``
    (paged like the cache, block table ``pool_table``).  ``gate`` float32 [T, >= H] (a view with any row stride):
    head h's output is multiplied by sigmoid(gate[t, h])."""
    _dev(q, out, k_cache, v_cache, block_table, token_seq, token_pos, pool_k, pool_v, pool_table, gate)
    _contig("out", out), _contig("block_table", block_table)
    if pool:
        _contig("pool_table", pool_table)
        assert pool_table.shape == block_table.shape and pool_k.dtype == k_cache.dtype == pool_v.dtype
        assert pool_k.is_contiguous() and pool_v.is_contiguous()
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    v_head_dim = v_head_dim or head_dim
    assert q.stride(1) == 1 and q.shape[1] >= n_heads * head_dim and out.shape[1] == n_heads * v_head_dim
    if head_dim > 256 or v_head_dim > 256:
        raise Unsupported(f"head_dim {head_dim}/{v_head_dim}: the general attention kernel takes sizes up to 256")
    if n_heads % n_kv_heads:
        raise Unsupported(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
    f = _fn("attention", "llmx_attention_paged_pooled",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_longlong, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p,
             c_void_p, c_void_p, c_void_p, c_longlong, c_void_p])
    _check(f(_ptr(q), _ptr(out), _tag(q), _ptr(k_cache), _ptr(v_cache), _tag(k_cache), _ptr(block_table),
             block_table.shape[1], _ptr(token_seq), _ptr(token_pos), q.shape[0], n_heads, n_kv_heads, head_dim,
             v_head_dim, q.stride(0), int(window or 0), int(keep_first or 0), scale, float(sink or 0.0), int(chunk or 0),
             int(pool or 0), _ptr(pool_k), _ptr(pool_v), _ptr(pool_table), _ptr(gate),
             gate.stride(0) if gate is not None else 0, _stream()), "attention_paged")


def pool_blocks(k_cache, v_cache, block_table, pool_k, pool_v, pool_table, seq_start, seq_past, n_seqs: int,
                n_tokens: int, n_kv_heads: int, head_dim: int, v_head_dim: int, pool: int) -> None:
    """For every block of ``pool`` positions whose last position the step brings (sequence s held ``seq_past[s]``
    positions and brings ``seq_start[s+1] - seq_start[s]``): the means of the block's keys and values, as the cache
    holds them, become row ``block`` of ``pool_k`` / ``pool_v``."""
    _dev(k_cache, v_cache, block_table, pool_k, pool_v, pool_table, seq_start, seq_past)
    _contig("block_table", block_table), _contig("pool_table", pool_table)
    assert pool_table.shape == block_table.shape and k_cache.dtype == v_cache.dtype == pool_k.dtype == pool_v.dtype
    assert all(t.is_contiguous() for t in (k_cache, v_cache, pool_k, pool_v))
    assert seq_start.numel() >= n_seqs + 1 and seq_past.numel() >= n_seqs
    f = _fn("attention", "llmx_pool_blocks",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p])
    _check(f(_ptr(k_cache), _ptr(v_cache), _tag(k_cache), _ptr(block_table), _ptr(pool_k), _ptr(pool_v),
             _ptr(pool_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, n_tokens, n_kv_heads,
             head_dim, v_head_dim, pool, k_cache.shape[0], pool_k.shape[0], _stream()), "pool_blocks")


def latent_norms(down, q_gain, kv_gain, eps: float, cq, c, q_rank: int, kv_rank: int) -> None:
    """The two latents of a latent attention out of its fused first product: ``down`` [T, >= q_rank + kv_rank]
    (or float32 split partials [S, T, ..]) -> cq = rms(down[:, :q_rank]) * q_gain, c = rms(down[:, q_rank :
    q_rank + kv_rank]) * kv_gain, float32 statistics, in the dtype of ``cq`` and ``c``."""
    _dev(down, q_gain, kv_gain, cq, c)
    _contig("down", down), _contig("cq", cq), _contig("c", c)
    n_split, stride = (down.shape[0], down.stride(0)) if down.dim() == 3 else (1, 0)
    T = down.shape[-2]
    assert cq.shape == (T, q_rank) and c.shape == (T, kv_rank) and cq.dtype == c.dtype
    assert q_gain.dtype == kv_gain.dtype == torch.float32 and q_gain.numel() == q_rank and kv_gain.numel() == kv_rank
    f = _fn("latent_attention", "llmx_latent_norms",
            [c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(down), _tag(down), n_split, stride, down.shape[-1], _ptr(q_gain), _ptr(kv_gain), eps, _ptr(cq),
             _ptr(c), _tag(cq), T, q_rank, kv_rank, _stream()), "latent_norms")


def latent_rope_cache(q, kv, down, k_rot_off: int, q_out, k_cache, v_cache, block_table, ctx, cos, sin, n_heads: int,
                      head_dim: int, rot_dim: int, v_head_dim: int) -> None:
    """Rotation and cache write of a latent attention.  q [T, H*(R+D)] (every head: rotated part, then unrotated),
    kv [T, H*D + H*Dv] (unrotated keys, then values), ``down`` as for ``latent_norms`` with the shared rotated key
    part at columns k_rot_off .. k_rot_off+R-1 -> q_out [T, H*(R+D)], one key [rot(shared) | unrotated] per head
    and the values into the paged cache entry [pages, H, PAGE, R+D] / [pages, H, PAGE, Dv]."""
    _dev(q, kv, down, q_out, k_cache, v_cache, block_table, cos, sin)
    for name, t in (("q", q), ("kv", kv), ("down", down), ("q_out", q_out), ("block_table", block_table)):
        _contig(name, t)
    n_split, stride = (down.shape[0], down.stride(0)) if down.dim() == 3 else (1, 0)
    T, H, D, R, Dv = q.shape[0], n_heads, head_dim, rot_dim, v_head_dim
    assert q.shape[1] == H * (R + D) == q_out.shape[1] and kv.shape == (T, H * (D + Dv)) and q.dtype == kv.dtype
    assert k_cache.shape[1:] == (H, PAGE, R + D) and v_cache.shape[1:] == (H, PAGE, Dv) and k_cache.dtype == v_cache.dtype
    assert cos.shape[1] == R // 2 and cos.dtype == torch.float32 and k_cache.is_contiguous() and v_cache.is_contiguous()
    f = _fn("latent_attention", "llmx_latent_rope_cache",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_int, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_longlong, c_void_p])
    _check(f(_ptr(q), _ptr(kv), _tag(q), _ptr(down), _tag(down), n_split, stride, down.shape[-1], k_rot_off,
             _ptr(q_out), _tag(q_out), _ptr(k_cache), _ptr(v_cache), _tag(k_cache), _ptr(block_table),
             block_table.shape[1], _ptr(ctx.token_seq), _ptr(ctx.token_pos), _ptr(cos), _ptr(sin), T, H, D, R, Dv,
             ctx.n_seqs, k_cache.shape[0], _stream()), "latent_rope_cache")


def head_gate(out, gate, n_heads: int, v_head_dim: int) -> None:
    """out[t, h, :] *= sigmoid(gate[t, h]) in place; out [T, H*Dv], gate float32 [T, >= H] (any row stride)."""
    _dev(out, gate)
    _contig("out", out)
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] >= n_heads
    assert out.shape[1] == n_heads * v_head_dim and gate.shape[0] == out.shape[0]
    f = _fn("latent_attention", "llmx_head_gate", [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _tag(out), _ptr(gate), gate.stride(0), out.shape[0], n_heads, v_head_dim, _stream()), "head_gate")


def n_sm(device=None) -> int:
    """Streaming multiprocessors of the device (asked once)."""
    from .parts.runtime import kernels_n_sm
    return kernels_n_sm(device if device is not None else "cuda")


def decode_chunks(n_seqs: int, n_kv_heads: int, group: int, n_pages: int, sms: int = 148) -> int:
    """Into how many shares the decode attention kernel cuts every sequence's
    visible keys.  A CTA (two warps) takes one share of one (sequence, kv head,
    8 query heads); two CTAs fit an SM, and the whole grid should be resident
    at once, so the shares are as many as that allows on ``sms`` multiprocessors,
    and never more than would leave a warp without a 32-key tile of a full block
    table.  Up to 8 shares the CTAs of a sequence and kv head merge as one
    thread-block cluster.  Beyond 8 (up to 32) the partials go through a
    workspace, which costs a little more per share; that is taken only where a
    small batch with a long context would otherwise leave most of the GPU idle:
    when 8 shares fill less than half of it and every share still has at least
    8 pages of keys.  It depends on the batch's shape only (not on its lengths),
    so a captured graph stays valid while the shape does; each sequence's own
    length is divided on the device."""
    base = n_seqs * n_kv_heads * ((group + 7) // 8)
    room = 2 * sms // base
    n = max(1, min(room, n_pages, 8))
    if n == 8 and base * 8 <= sms:
        n = max(8, min(3 * sms // (2 * base), n_pages // 8, 32))     # about one and a half CTAs per SM measured best
    return n


_decode_counters: dict = {}


def _counters(device, n: int):
    """Zeroed arrival counters for kernels whose last CTA finishes a reduction;
    every launch leaves them zero, so one buffer per device serves all calls."""
    buf = _decode_counters.get(device)
    if buf is None or buf.numel() < n:
        buf = guard.guarded((max(n, 16384),), torch.int32, device, "decode attention counters", zero=True)
        _decode_counters[device] = buf
    return buf


def attention_decode(q, out, k_cache, v_cache, block_table, seq_past, n_heads: int, n_kv_heads: int,
                     head_dim: int, window, scale: float, n_chunks: int = 0, keep_first: int = 0,
                     sink: float = 0.0, chunk: int = 0, pool: int = 0, pool_k=None, pool_v=None, pool_table=None) -> None:
    """One new token per sequence, bfloat16: q, out [B,H*D] in batch order;
    seq_past[b] is the token's position.  Each sequence's keys are split over
    n_chunks CTAs (0: chosen from the batch's shape), which merge inside a
    cluster, or beyond 8 chunks through a float32 workspace.  ``chunk`` n > 0 is
    the chunked mask of ``attention_paged`` (nothing to do with n_chunks); ``pool`` with its second store likewise."""
    _dev(q, out, k_cache, v_cache, block_table, seq_past, pool_k, pool_v, pool_table)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    if pool:
        _contig("pool_table", pool_table)
        assert pool_table.shape == block_table.shape and pool_k.dtype == pool_v.dtype == torch.bfloat16
        assert pool_k.is_contiguous() and pool_v.is_contiguous() and pool_k.shape[1:] == k_cache.shape[1:]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    if head_dim % 16 or head_dim > 256:
        raise Unsupported(f"head_dim {head_dim}: the decode attention kernel takes multiples of 16 up to 256")
    B = q.shape[0]
    n_pages = block_table.shape[1]
    if window and pool:       # the window's pages and the pages of block rows that a full table can hold
        n_pages = min(n_pages, (window + PAGE - 2) // PAGE + 1 + (n_pages + int(pool) - 1) // int(pool))
    elif window:
        n_pages = min(n_pages, (window + PAGE - 2) // PAGE + 1 + (int(keep_first or 0) + PAGE - 1) // PAGE)
    if chunk:
        n_pages = min(n_pages, (int(chunk) + PAGE - 1) // PAGE + 1)
    group = n_heads // n_kv_heads
    n_chunks = n_chunks or decode_chunks(B, n_kv_heads, group, n_pages, n_sm(q.device))
    ws = counters = None
    if n_chunks > 8:
        ws = guard.scratch((B * n_heads * n_chunks * (head_dim + 4),), torch.float32, q.device,
                           "decode attention workspace")
        counters = _counters(q.device, B * n_kv_heads * ((group + 7) // 8))
    f = _fn("attention_decode", "llmx_attention_decode_pooled",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p, c_longlong,
             c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
             block_table.shape[1],
             _ptr(seq_past), _ptr(ws), _ptr(counters), B, n_heads, n_kv_heads, head_dim, int(window or 0),
             int(keep_first or 0), int(chunk or 0), scale, float(sink or 0.0), n_chunks, int(pool or 0), _ptr(pool_k),
             _ptr(pool_v), pool_k.shape[0] if pool else 0, _ptr(pool_table), _stream()), "attention_decode")


def attention_decode_status() -> int:
    """0, or 1 after a decode attention launch whose shared-memory copies never completed."""
    lib = load_library("attention_decode")
    lib.llmx_attention_decode_status.restype = c_int
    return int(lib.llmx_attention_decode_status())


def attention_prefill_supports(q, k_cache, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim in (64, 128)


def attention_prefill(q, out, k_cache, v_cache, block_table, seq_start, seq_past, n_seqs: int, max_new: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, window, scale: float, keep_first: int = 0,
                      sink: float = 0.0, chunk: int = 0, pool: int = 0, pool_k=None, pool_v=None, pool_table=None) -> None:
    """Prompt attention on the tensor cores, bfloat16, head sizes 64 and 128:
    q, out [T,H*D] packed sequence after sequence.  Under a window the first ``keep_first`` keys stay visible;
    ``chunk`` n > 0 is the chunked mask of ``attention_paged``, ``pool`` with its second store its pooled blocks."""
    _dev(q, out, k_cache, v_cache, block_table, seq_start, seq_past, pool_k, pool_v, pool_table)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    if pool:
        _contig("pool_table", pool_table)
        assert pool_table.shape == block_table.shape and pool_k.dtype == pool_v.dtype == torch.bfloat16
        assert pool_k.is_contiguous() and pool_v.is_contiguous() and pool_k.shape[1:] == k_cache.shape[1:]
    if not attention_prefill_supports(q, k_cache, head_dim):
        raise Unsupported(f"the tiled prompt attention takes bfloat16 and head sizes 64 or 128, not {head_dim}")
    f = _fn("attention_prefill", "llmx_attention_prefill_pooled",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(seq_start), _ptr(seq_past), n_seqs, max_new, n_heads, n_kv_heads, head_dim, int(window or 0),
             int(keep_first or 0), int(chunk or 0), scale, float(sink or 0.0), int(pool or 0), _ptr(pool_k), _ptr(pool_v),
             _ptr(pool_table), _stream()), "attention_prefill")


def attention_prefill_tc(q, out, k_cache, v_cache, block_table, seq_start, seq_past, n_seqs: int, max_new: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, window, scale: float, keep_first: int = 0,
                         sink: float = 0.0, chunk: int = 0) -> None:
    """Prompt attention on tcgen05, bfloat16, head size 128: q, out [T,H*128]
    packed sequence after sequence; the cache entry is [n_pages,G,64,128].  ``chunk`` n > 0 is the chunked mask
    of ``attention_paged``."""
    _dev(q, out, k_cache, v_cache, block_table, seq_start, seq_past)
    _contig("q", q), _contig("out", out), _contig("block_table", block_table)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    if head_dim != 128 or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise Unsupported("the tcgen05 prompt attention takes bfloat16 and head size 128")
    f = _fn("attention_prefill_tc", "llmx_attention_prefill_tc_masked",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table),
             block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, q.shape[0], max_new, n_heads,
             n_kv_heads, head_dim, int(window or 0), int(keep_first or 0), int(chunk or 0), scale, float(sink or 0.0),
             _stream()), "attention_prefill_tc")


def attention_prefill_tc_status(reset: bool = True) -> int:
    """0, or which bounded wait of the tcgen05 prompt attention ran out.  Synchronises the device."""
    f = _fn("attention_prefill_tc", "llmx_attention_prefill_tc_status", [c_int])
    return f(int(reset))


def gemm_fma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = x[M,K] @ w[N,K]^T on the FMA units, float32 accumulation in
    the order k = 0..K-1.  Rows may be strided; the K axis must be dense."""
    _dev(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    f = _fn("gemm_fma", "llmx_gemm_fma",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
             c_longlong, c_void_p])
    _check(f(_ptr(x), _tag(x), _ptr(w), _tag(w), _ptr(out), _tag(out), M, N, K, x.stride(0), w.stride(0),
             out.stride(0), _stream()), "gemm_fma")


PAIR_MIN_TOKENS = 128      # the CTA-pair kernel (tcgen05 cta_group::2) takes steps of more tokens than this


def gemm_tc_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the tensor-core kernel takes: bfloat16, dense K axis, K and the
    row strides multiples of 8 elements (TMA wants 16-byte strides and starts)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_gated_supports(activation) -> bool:
    """Whether the tensor-core product applies this gated activation in its epilogue."""
    return (activation if isinstance(activation, str) else activation[0]) in GATE_ACTS


_tc_gate_act = [("silu",)]        # what the gemm_tc library was last told


def _set_tc_gate_act(activation) -> None:
    """The gated activation of the tensor-core launches that follow (a kernel argument, set on the host)."""
    key = gate_act_args(activation)
    if _tc_gate_act[0] != key:
        f = _fn("gemm_tc", "llmx_gemm_tc_gate_act", [c_int, c_float, c_float, c_float])
        code = f(*key)
        if code:
            raise Unsupported(f"gemm_tc: activation {activation!r} refused")
        _tc_gate_act[0] = key


_tc_gate_bias = [0]               # the bias pointer the gemm_tc library was last told (0: none)
TC_BIAS_PAD = 256                 # a gated launch's bias covers whole row tiles of a CTA pair


def _set_tc_gate_bias(bias) -> None:
    """The bias of the gated tensor-core launches that follow (a kernel argument, set on the host); None: none."""
    ptr = 0 if bias is None else bias.data_ptr()
    if _tc_gate_bias[0] != ptr:
        f = _fn("gemm_tc", "llmx_gemm_tc_gate_bias", [c_void_p])
        f(ptr or None)
        _tc_gate_bias[0] = ptr


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_split: int = 1, gated=False,
            pair: bool = False, scale=None, accumulate: bool = False, activation="silu", gate_bias=None) -> None:
    """bfloat16 x [T,K] times w [N,K]^T on tcgen05.  ``out`` is [T,N] (bfloat16
    or float32), or float32 partials [n_split,T,N] of a split reduction, or,
    with ``gated``, [T,N/2] = silu(gate) * up: ``gated=True`` (or 1) for
    w = [gate rows; up rows], ``gated=2`` for w in blocks of 16 gate rows each
    followed by the 16 up rows of the same features (N/2 a multiple of 16).
    ``pair`` runs the CTA-pair kernel (prompt-sized T > 128; it splits too); with
    ``accumulate`` it adds to a float32 ``out`` instead of overwriting it
    (one float32 addition per element, whatever order the tiles finish in).
    ``scale = (sumsq, parts, eps, d)``, for T <= 64: output row t is multiplied
    by 1/sqrt(sum(sumsq[:parts, t]) / d + eps) before any activation (the
    second half of an RMSNorm whose first half is ``add_gain_sumsq``).
    ``gate_bias`` (``gated=2`` only): float32, one per row of w in w's row order, zero-padded to a multiple of
    ``TC_BIAS_PAD`` rows; added to the products before the activation."""
    gated = int(gated)
    _dev(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.is_contiguous()
    if gated:
        if not gemm_tc_gated_supports(activation):
            raise Unsupported(f"the tensor-core product has no epilogue for the activation {activation!r}")
        _set_tc_gate_act(activation)
        if gate_bias is not None:
            _dev(gate_bias)
            assert gated == 2 and gate_bias.dtype == torch.float32 and gate_bias.is_contiguous()
            assert gate_bias.numel() >= (N + TC_BIAS_PAD - 1) // TC_BIAS_PAD * TC_BIAS_PAD
        _set_tc_gate_bias(gate_bias)
    else:
        assert gate_bias is None
    if gated:
        assert n_split == 1 and out.shape == (T, N // 2)
        ldy, stride = N // 2, 0
    elif n_split > 1:
        assert out.shape == (n_split, T, N) and out.dtype == torch.float32
        ldy, stride = N, out.stride(0)
    else:
        assert out.shape == (T, N)
        ldy, stride = N, 0
    assert pair or not accumulate
    if pair:
        assert T > PAIR_MIN_TOKENS and scale is None and not (accumulate and n_split > 1)
        f = _fn("gemm_tc", "llmx_gemm_tc_pair",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                 c_int, c_int, c_longlong, c_void_p])
        _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy,
                 gated, int(accumulate), n_split, stride, _stream()), "gemm_tc_pair")
        return
    if scale is None:
        f = _fn("gemm_tc", "llmx_gemm_tc",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                 c_longlong, c_int, c_void_p])
        _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy, n_split, stride,
                 gated, _stream()), "gemm_tc")
        return
    sumsq, parts, eps, d = scale
    _dev(sumsq)
    assert T <= 64 and sumsq.dtype == torch.float32 and sumsq.shape[0] >= parts and sumsq.stride(1) == 1
    f = _fn("gemm_tc", "llmx_gemm_tc_scaled",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
             c_longlong, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(out), _tag(out), T, N, K, x.stride(0), w.stride(0), ldy, n_split, stride, gated,
             _ptr(sumsq), parts, sumsq.stride(0), eps, d, _stream()), "gemm_tc (row scales)")


def gemm_tc_status(reset: bool = True) -> int:
    """0, or which role of the tensor-core kernel ran out of its bounded wait
    since the last reset.  Synchronises the device."""
    f = _fn("gemm_tc", "llmx_gemm_tc_status", [c_int])
    return f(int(reset))


def fill_normal(out: torch.Tensor, stream: int, quantiles: torch.Tensor, mean: float, std: float,
                storage_dtype: torch.dtype) -> None:
    """out[i] = mean + std * normal(stream, i), rounded to ``storage_dtype`` first: the counter-based
    generator of ``weights.random_init`` (same bits as its host version)."""
    _dev(out, quantiles)
    _contig("out", out)
    assert quantiles.dtype == torch.float32 and quantiles.numel() == 65537 and quantiles.is_contiguous()
    f = _fn("random_init", "llmx_fill_normal",
            [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_void_p, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(out), _tag(out), out.numel(), stream & 0xFFFFFFFFFFFFFFFF, _ptr(quantiles), mean, std,
             _DTYPE_TAG[storage_dtype], _stream()), "fill_normal")


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor) -> None:
    """out_tokens[b] = the last index among the maxima of logits[b,:]."""
    _dev(logits, out_tokens)
    assert logits.dtype == torch.float32 and out_tokens.dtype == torch.int32 and logits.stride(1) == 1
    f = _fn("sampling", "llmx_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(out_tokens), _stream()),
           "argmax")


def sample(logits, temperature, top_k, top_p, repeat_penalty, recent, uniform, out_tokens, status) -> None:
    """One token per row of float32 ``logits`` [B,V] (changed in place by the
    repetition penalty).  Per-row parameters are device tensors [B]; ``recent``
    is int32 [B,W] with -1 for no token, or None.  ``status`` int32 [1] (on the
    device or page-locked on the host) is set non-zero when a row asked for what
    the kernel cannot do."""
    _dev(logits, temperature, top_k, top_p, repeat_penalty, recent, uniform, out_tokens)
    if not (status.is_cuda or status.is_pinned()):
        raise KernelError("the sampler's status word must be on the GPU or in page-locked host memory")
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert top_k.dtype == torch.int32 and out_tokens.dtype == torch.int32 and status.dtype == torch.int32
    f = _fn("sampling", "llmx_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p])
    width = 0 if recent is None else recent.shape[1]
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(repeat_penalty), _ptr(recent), width, _ptr(uniform), _ptr(out_tokens),
             _ptr(status), _stream()), "sample")


# ---- linear attention with a decay ---------------------------------------------------------------------

_ACTS = {"none": 0, "silu": 1, "sigmoid": 2}


def _split_view(proj):
    """(n_split, split stride, row stride) of a product's output: [T, N], or float32 partials [S, T, N]."""
    assert proj.stride(-1) == 1
    if proj.dim() == 3:
        return proj.shape[0], proj.stride(0), proj.stride(1)
    return 1, 0, proj.stride(0)


def decay_scan(proj, out, state, seq_start, token_pos, seq_slot, decay, cos, sin, n_rot: int, activation: str,
               k_scale: float, n_heads: int, head_dim: int, v_head_dim: int, q_off: int, k_off: int, v_off: int,
               max_new: int = 0, seg_len: int = 0, gates=None, q_scale: float = 1.0, ones_column: bool = False) -> None:
    """The recurrence S = decay_h S + k v^T, o = S^T q over every sequence's tokens of the step, in order.
    ``proj`` [T, N] (or split partials [S, T, N]) holds q heads at column ``q_off``, k heads at ``k_off``
    (``head_dim`` each) and v heads at ``v_off`` (``v_head_dim`` each); ``activation`` is applied to all three,
    then q and k are rotated (first ``n_rot`` dims, float32 tables, at ``token_pos``) and scaled.  ``out`` float32
    [T, H*Dv]; ``state`` float32 [slots, H, D, Dv], read and written in place for the step's slots.  A sequence
    that brings more than ``seg_len`` tokens (0: 128) is walked in segments side by side; ``max_new`` is the most
    tokens one sequence brings (0: not known, taken as all of them).

    With ``gates`` (float32 [T, H, 4] as ``gate_scan`` leaves them, same ``seg_len``) decay and input weight come
    per token: S_t = a_t S_(t-1) + b_t k_t v_t^T.  With ``ones_column`` the values get one more column that is 1
    for every token (its state column is the sum of the weighted keys, its output q . that sum): ``out`` is then
    [T, H*(Dv+1)], and ``state`` [slots, H, n] with n >= D*(Dv+1) floats a head, S first."""
    _dev(proj, out, state, seq_start, token_pos, seq_slot, decay, cos, sin, gates)
    _contig("out", out), _contig("state", state)
    assert out.dtype == torch.float32 and state.dtype == torch.float32
    assert decay is None or (decay.dtype == torch.float32 and decay.numel() == n_heads)
    assert gates is not None or decay is not None
    dva = v_head_dim + (1 if ones_column else 0)
    assert out.shape[1] == n_heads * dva and state.shape[1] == n_heads
    head_stride = state.stride(1)
    assert head_stride >= head_dim * dva
    n_split, split_stride, row_stride = _split_view(proj)
    n_seqs, T = seq_slot.numel(), out.shape[0]
    assert gates is None or (gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape == (T, n_heads, 4))
    pad4 = lambda n: (n + 3) // 4 * 4
    # q, k and v of every (token, head) after activation, rotation and scale, float32, rows padded to 4 elements
    prep = guard.scratch((T * n_heads * (2 * pad4(head_dim) + pad4(dva)),), torch.float32, out.device,
                         "prepared q, k, v of the recurrence")
    max_new = max_new if 0 < max_new <= T else T
    seg = seg_len or 128
    n_seg = (max_new + seg - 1) // seg
    partial = None
    if n_seg > 1:
        partial = guard.scratch((n_seqs * n_heads * n_seg * head_dim * dva,), torch.float32, out.device,
                                "last states of a prompt's segments")
    f = _fn("linear_attention", "llmx_decay_scan",
            [c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_float, c_int, c_void_p])
    _check(f(_ptr(proj), _tag(proj), n_split, split_stride, row_stride, q_off, k_off, v_off, _ptr(prep), _ptr(out),
             _ptr(state), _ptr(partial), _ptr(seq_start), _ptr(token_pos), _ptr(seq_slot), _ptr(decay), _ptr(cos),
             _ptr(sin), n_rot, _ACTS[activation], k_scale, T, n_seqs, max_new, seg, n_heads, head_dim, v_head_dim,
             n_sm(out.device), _ptr(gates), head_stride, q_scale, int(ones_column), _stream()), "decay_scan")
    global launch_count
    launch_count += 2 if n_seg > 1 else 1          # beside the preparation: the recurrence, and the segments' second pass


def gate_scan(proj, i_off: int, f_off: int, bias_i, bias_f, cap: float, gates, state, m_off: int, seq_start, seq_slot,
              n_heads: int, seg_len: int = 0) -> None:
    """The gates of a recurrence with a running maximum, per (sequence, head) over the step's tokens in order:
    i = cap tanh((proj[:, i_off + h] + bias_i[h]) / cap), f = logsigmoid(cap tanh((proj[:, f_off + h] + bias_f[h]) /
    cap)) (``cap`` <= 0: no cap), m_t = max(f_t + m_(t-1), i_t).  ``gates`` float32 [T, H, 4] receives a_t =
    exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t), exp(-m_t) and the product of a over the token's segment so far
    (segments of ``seg_len`` tokens, 0: 128, counted from the sequence's first token of the step).  m lives in
    ``state`` [slots, H, n] at ``m_off`` floats into a head's state and is moved on in place."""
    _dev(proj, bias_i, bias_f, gates, state, seq_start, seq_slot)
    _contig("gates", gates), _contig("state", state)
    assert gates.dtype == torch.float32 and state.dtype == torch.float32 and state.shape[1] == n_heads
    assert all(b is None or (b.dtype == torch.float32 and b.numel() == n_heads and b.is_contiguous()) for b in (bias_i, bias_f))
    n_split, split_stride, row_stride = _split_view(proj)
    f = _fn("linear_attention", "llmx_gate_scan",
            [c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
             c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), _tag(proj), n_split, split_stride, row_stride, i_off, f_off, _ptr(bias_i), _ptr(bias_f),
             float(cap or 0.0), _ptr(gates), _ptr(state), state.stride(1), m_off, _ptr(seq_start), _ptr(seq_slot),
             seq_slot.numel(), n_heads, seg_len or 128, _stream()), "gate_scan")


def gated_norm(o, proj, g_off: int, gain, eps: float, gate: str, per_head: bool, y, n_heads: int,
               v_head_dim: int, gates=None, den_eps: float = 0.0) -> None:
    """y = o / sqrt(mean(o^2) + eps) * gain * gate(proj[:, g_off:]) with the mean over one head's columns
    (``per_head``) or over the whole row; o float32 [T, H*Dv]; ``gain`` float32 [H*Dv] or None.  With ``gates``
    (``gate_scan``'s, per_head only) o is [T, H*(Dv+1)], a head's last column being n . q, and o is first divided
    by max(|n . q|, exp(-m)) + ``den_eps``."""
    _dev(o, proj, gain, y, gates)
    _contig("o", o), _contig("y", y)
    assert o.dtype == torch.float32 and (gain is None or gain.dtype == torch.float32)
    assert y.shape == (o.shape[0], n_heads * v_head_dim)
    assert o.shape[1] == n_heads * (v_head_dim + (1 if gates is not None else 0))
    n_split, split_stride, row_stride = _split_view(proj)
    f = _fn("linear_attention", "llmx_gated_norm",
            [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_float, c_int, c_int, c_void_p,
             c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p])
    _check(f(_ptr(o), _ptr(proj), _tag(proj), n_split, split_stride, row_stride, g_off, _ptr(gain), eps, _ACTS[gate],
             int(per_head), _ptr(y), _tag(y), o.shape[0], n_heads, v_head_dim, _ptr(gates), den_eps, _stream()),
           "gated_norm")


# ---- routed experts ------------------------------------------------------------------------------------

MOE_TILE = 64          # rows per tile of the grouped products; the same constant as in moe.cu
_SCORES = {"sigmoid": 0, "softmax": 1, "softmax_top": 2}


def moe_route(logits, ids, weights, top: int, n_groups: int, keep_groups: int, group_top: int, score: str,
              normalize: bool, norm_eps: float, scale: float, bias=None) -> None:
    """Per token (row of float32 ``logits`` [T, E]): its ``top`` experts (``ids`` int32 [T, top]) and their
    weights (float32 [T, top]); see moe.cu for the rule.  ``bias`` float32 [E]: a correction added to the scores
    for the choice only."""
    _dev(logits, ids, weights, bias)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == logits.shape[1] and bias.is_contiguous())
    _contig("logits", logits), _contig("ids", ids), _contig("weights", weights)
    assert logits.dtype == torch.float32 and ids.dtype == torch.int32 and weights.dtype == torch.float32
    T, E = logits.shape
    f = _fn("moe", "llmx_moe_route",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
             c_void_p, c_void_p])
    _check(f(_ptr(logits), _ptr(ids), _ptr(weights), T, E, top, n_groups, keep_groups, group_top, _SCORES[score],
             int(normalize), norm_eps, scale, _ptr(bias), _stream()), "moe_route")


def moe_table_route(tokens, table, n_experts: int, weight: float, ids, weights) -> None:
    """Routing by a table: token t's experts are row ``tokens[t]`` of the int32 ``table`` [vocab, top], each with
    ``weight``; -> ids int32 [T, top], weights float32 [T, top]."""
    _dev(tokens, table, ids, weights)
    _contig("table", table), _contig("ids", ids), _contig("weights", weights), _contig("tokens", tokens)
    assert table.dtype == torch.int32 and tokens.dtype == torch.int32 and ids.dtype == torch.int32
    assert weights.dtype == torch.float32 and ids.shape == weights.shape == (tokens.numel(), table.shape[1])
    f = _fn("moe", "llmx_moe_table_route",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(tokens), _ptr(table), table.shape[0], n_experts, table.shape[1], weight, _ptr(ids), _ptr(weights),
             tokens.numel(), _stream()), "moe_table_route")


def moe_max_tiles(n_pairs: int, n_experts: int, tile_rows: int = MOE_TILE) -> int:
    return (n_pairs + tile_rows - 1) // tile_rows + n_experts


def moe_sort(ids, n_experts: int, perm, tiles, tile_rows: int = MOE_TILE, pair_weight=None, dest=None,
             sorted_weight=None, n_tiled=None) -> None:
    """Orders the (token, choice) pairs by expert: ``perm`` int32 [P] (sorted place -> pair) and ``tiles``
    int32 [max_tiles, 3] (expert or -1, first row, rows), of up to ``tile_rows`` rows each.  With ``dest`` and
    ``sorted_weight`` ([P]) also, in sorted order, the row choice * T + token where a pair's result goes and the
    pair's weight (``pair_weight`` [T, top]).  Experts from ``n_tiled`` on (identity experts) get no tiles."""
    _dev(ids, perm, tiles, pair_weight, dest, sorted_weight)
    _contig("ids", ids), _contig("perm", perm), _contig("tiles", tiles)
    T, top = ids.shape
    f = _fn("moe", "llmx_moe_sort", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(pair_weight), ids.numel(), n_experts, top, T, _ptr(perm), _ptr(dest), _ptr(sorted_weight),
             _ptr(tiles), tiles.shape[0], tile_rows, n_experts if n_tiled is None else n_tiled, _stream()), "moe_sort")


def moe_router(x, w, ids, weights, n_groups: int, keep_groups: int, group_top: int, score: str, normalize: bool,
               norm_eps: float, scale: float, bias=None, extra_out=None, logit_bias=None) -> None:
    """The router's product (float32 ``w`` [E, K] times the rows of ``x``, float32 sums) and the routing of
    ``moe_route`` in one kernel.  With ``extra_out`` float32 [T, n], ``w`` holds n more rows behind the experts',
    whose products are written there as they are.  ``logit_bias`` float32 [E] joins the experts' logits before the
    scores are made.  ``score`` "softmax_top": the largest logits win, and the weights are the softmax over the
    winners' logits only."""
    _dev(x, w, ids, weights, bias, extra_out, logit_bias)
    assert logit_bias is None or (logit_bias.dtype == torch.float32 and logit_bias.is_contiguous()
                                  and logit_bias.numel() == w.shape[0] - (0 if extra_out is None else extra_out.shape[1]))
    n_extra = 0 if extra_out is None else extra_out.shape[1]
    assert extra_out is None or (extra_out.dtype == torch.float32 and extra_out.is_contiguous())
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == w.shape[0] - n_extra and bias.is_contiguous())
    _contig("w", w), _contig("ids", ids), _contig("weights", weights)
    assert w.dtype == torch.float32 and x.stride(1) == 1 and ids.dtype == torch.int32 and weights.dtype == torch.float32
    T, top = ids.shape
    f = _fn("moe", "llmx_moe_router_biased",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(x), _tag(x), x.stride(0), _ptr(w), _ptr(ids), _ptr(weights), T, x.shape[1], w.shape[0] - n_extra, top,
             n_groups, keep_groups, group_top, _SCORES[score], int(normalize), norm_eps, scale, _ptr(bias), n_extra,
             _ptr(extra_out), _ptr(logit_bias), _stream()), "moe_router")


def moe_tc_supports(x, w) -> bool:
    """Shapes the tensor-core grouped product takes: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous()
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_tc_gated_supports(activation) -> bool:
    """Whether the tensor-core grouped product applies this gated activation in its epilogue."""
    return (activation if isinstance(activation, str) else activation[0]) in GATE_ACTS


def moe_gather_rows(x, perm, top: int, xs) -> None:
    """xs[place] = x[perm[place] // top]: the tokens' rows in the sorted order of their pairs (bfloat16)."""
    _dev(x, perm, xs)
    _contig("xs", xs)
    assert x.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and xs.shape == (perm.numel(), x.shape[1])
    f = _fn("moe_tc", "llmx_moe_gather_rows", [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(perm), top, _ptr(xs), perm.numel(), x.shape[1], _stream()), "moe_gather_rows")


def moe_grouped_tc(xs, w, y, tiles, tile_rows: int, dest, sorted_weight, gated: bool, activation="silu") -> None:
    """The grouped products on tcgen05.  ``xs`` bfloat16 [P, K] in sorted order; ``gated``: w [E, 2F, K] (gate rows,
    then up rows), y bfloat16 [P, F]; else w [E, N, K], y float32 [top, T, N] whose row ``dest[place]`` becomes
    ``sorted_weight[place]`` times the product.  ``tiles`` made by ``moe_sort`` with ``tile_rows`` in (16, 64, 128)."""
    _dev(xs, w, y, tiles, dest, sorted_weight)
    _contig("w", w), _contig("y", y)
    assert moe_tc_supports(xs, w) and tile_rows in (16, 64, 128) and (not gated or moe_tc_gated_supports(activation))
    K = xs.shape[1]
    N = w.shape[1] // 2 if gated else w.shape[1]
    assert w.shape[2] == K and y.dtype == (torch.bfloat16 if gated else torch.float32)
    f = _fn("moe_tc", "llmx_moe_grouped_tc",
            [c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(_ptr(xs), xs.stride(0), xs.shape[0], _ptr(w), w.shape[0], _ptr(y), _ptr(tiles), tiles.shape[0], tile_rows,
             _ptr(dest), _ptr(sorted_weight), N, K, int(gated), *gate_act_args(activation), _stream()), "moe_grouped_tc")


def moe_grouped(x, w, y, perm, tiles, pair_weight, top: int, n_tokens: int, gated: bool, activation="silu") -> None:
    """Grouped products over the sorted pairs on the FMA units (the float32 path, and sizes the tensor-core kernel
    does not take).  ``gated``: x [T, K] gathered through ``perm``, w [E, 2F, K] (gate rows, then up rows), y [P, F] =
    silu(gate) * up in sorted order.  Else: x [P, K] in sorted order, w [E, N, K], y float32 [top, T, N] = weight of
    the pair times the product.  ``tiles`` made by ``moe_sort`` with ``MOE_TILE`` rows per tile."""
    _dev(x, w, y, perm, tiles, pair_weight)
    _contig("w", w), _contig("y", y)
    assert x.stride(1) == 1 and x.dtype == w.dtype
    K = x.shape[1]
    N = w.shape[1] // 2 if gated else w.shape[1]
    assert w.shape[2] == K
    f = _fn("moe", "llmx_moe_grouped_fma",
            [c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(_ptr(x), _tag(x), x.stride(0), _ptr(w), _tag(w), _ptr(y), _tag(y), _ptr(perm), _ptr(tiles), tiles.shape[0],
             _ptr(pair_weight), top, n_tokens, N, K, int(gated), *gate_act_args(activation), _stream()), "moe_grouped")


def moe_extras(x, ids, weights, y, n_real: int, shared=None, shared_z=None) -> None:
    """What the grouped products leave out, in one launch.  Identity experts: y[choice, t, :] = weights[t, choice] *
    x[t, :] for every pair whose expert id is ``n_real`` or more (an identity expert's output is its input); the other
    pairs' rows are left alone.  A shared expert: y[top, t, :] = sigmoid(shared_z[t]) * shared[t, :], or shared[t, :] itself without ``shared_z`` (``shared``
    [T, d] or partials [P, T, d]; ``shared_z`` float32, one number per token, a column of a wider row allowed).
    y float32 [top (+1), T, d]."""
    _dev(x, ids, weights, y, shared, shared_z)
    _contig("ids", ids), _contig("weights", weights), _contig("y", y)
    T, top = ids.shape
    d = x.shape[1]
    assert x.stride(1) == 1 and y.dtype == torch.float32 and y.shape[-2:] == (T, d)
    assert y.shape[0] >= top + (1 if shared is not None else 0)
    n_split, stride, stag, ldz = 1, 0, F32, 1
    if shared is not None:
        _contig("shared", shared)
        if shared.dim() == 2:
            shared = shared.unsqueeze(0)
        assert shared.shape[1:] == (T, d)
        assert shared_z is None or (shared_z.dtype == torch.float32 and shared_z.dim() == 1 and shared_z.numel() == T)
        n_split, stride, stag = shared.shape[0], shared.stride(0), _tag(shared)
        ldz = 1 if shared_z is None else shared_z.stride(0)
    f = _fn("moe", "llmx_moe_extras",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
             c_longlong, c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), _tag(x), x.stride(0), _ptr(ids), _ptr(weights), _ptr(y), T, top, d, n_real, _ptr(shared), stag,
             n_split, stride, _ptr(shared_z), ldz, _stream()), "moe_extras")
