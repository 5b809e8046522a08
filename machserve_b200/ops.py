"""Python face of the CUDA kernels: loads the library and wraps each entry point.

There is no CPU fallback and no library model code here.  If the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call fails loudly.
Wrappers check dtypes and shapes, pass raw pointers and the current stream, and
raise `KernelError` with the entry point's own message on a non-zero return.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None      # the loaded library (ctypes), behind `_proxy`
_files = None    # the source files whose kernels it holds: a set, or ALL
_flavor = None
ALL = "all"
# what every model needs whatever its parts: the error channel and launch switch, the stream's own kernels, the products
CORE_FILES = ("elementwise", "gemm_f32", "gemm_small_m")


def use_flavor(flavor) -> None:
    """Chooses another build of the kernels (csrc/build.py FLAVORS) for this process; before the library is first used."""
    global _flavor
    if _lib is not None and flavor != _flavor:
        raise KernelError("the kernel library is loaded already; choose the flavor before the first kernel call")
    _flavor = flavor


def _load(path) -> None:
    global _lib
    try:
        L = ctypes.CDLL(str(path))
    except OSError as e:
        raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
    L.ms_last_error.restype = ctypes.c_char_p
    for name in dir(_Signatures):
        if name.startswith("ms_"):
            try:
                fn = getattr(L, name)
            except AttributeError:
                continue  # a library of some of the files
            fn.argtypes = getattr(_Signatures, name)
            fn.restype = c_int
    L._ms_path = str(path)
    _lib = L


def require(files=None) -> None:
    """Makes sure that the loaded library holds the kernels of the named source files (names without `.cu`; None: of all
    files), building it first if need be.  A model's runner names the files its parts declare (`Part.kernel_files`), so that
    the first use of a model waits for the compilation of what it needs and of nothing else; where the whole library is
    there already, it is loaded whatever is asked.  A later call that asks for more loads a library of both."""
    global _files
    if _lib is not None and (_files == ALL or (files is not None and set(files) <= _files)):
        return
    want = None
    if files is not None:
        want = set(files) | set(CORE_FILES) | (_files if isinstance(_files, set) else set())
    path = _build.library_for(sorted(want) if want is not None else None, flavor=_flavor)
    _load(path)
    _files = ALL if want is None or path.name == _build.LIB_NAME else want


def has(name: str) -> bool:
    """Whether the loaded library holds the entry point `name` (a library of some of the files may not)."""
    return _lib is not None and hasattr(_lib, name)


class _Proxy:
    """The loaded library; an entry point that a library of some of the files lacks brings in the whole library."""

    def __getattr__(self, name):
        if _lib is None:
            require(None)
        try:
            return getattr(_lib, name)
        except AttributeError:
            if _files == ALL:
                raise
            require(None)
            return getattr(_lib, name)


_proxy = _Proxy()


def lib():
    """The loaded kernel library (built on first use: the whole of it, unless `require` named files before)."""
    if _lib is None:
        require(None)
    return _proxy


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it (on by default)."""
    lib().ms_set_pdl(1 if on else 0)


def library_file() -> str:
    lib()
    return _lib._ms_path


class _Signatures:
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    ms_embed_gather = [P, I, P, P, I, I, I, P]
    ms_add_rmsnorm = [P, P, I, P, P, I, P, I, I, F, P]
    ms_add_bias = [P, I, P, I, I, I, P]
    ms_silu_mul = [P, P, I, I, I, P]
    ms_add_layernorm = [P, P, I, P, I, P, P, P, P, P, P, I, P, I, I, F, P]
    ms_concat_streams = [P, P, I, P, I, P, P, I, I, I, P]
    ms_glu_clamped = [P, P, I, I, I, F, F, F, P]
    ms_sigmoid_gate_mul = [P, I, P, I, P, I, I, I, P]
    ms_qk_norm_store = [P, I, P, P, F, F, I, P, P, P, I, I, I, P, P, P, P, I, I, I, I, I, I, I, P]
    ms_latent_encode = [P, I, I, P, I, P, F, P, I, I, I, P, P, P, I, I, I, P, P, I, P, I, I, I, I, I, I, I, P]
    ms_embed_scaled_pos = [P, I, P, P, P, P, I, I, I, I, F, P]
    ms_add_streams_rmsnorm = [P, P, I, P, I, P, P, P, P, I, P, I, I, F, F, P]
    ms_norm_pair_mean = [P, P, P, P, P, I, I, F, F, P]
    ms_pair_weighted_sum = [P, P, P, P, P, I, I, F, F, P]
    ms_mm_gates = [P, I, I, I, P, P, F, P, LL, LL, P, P, P, P, I, I, P]
    ms_mm_scan = [P, I, I, I, I, P, F, P, LL, P, P, P, P, I, I, I, I, I, P]
    ms_mm_output = [P, P, P, I, P, F, P, I, I, I, I, P]
    ms_softcap = [P, LL, F, P]
    ms_head_gate_mul = [P, P, I, P, I, I, I, I, P]
    ms_rope_store = [P, I, P, P, I, I, I, P, P, P, I, I, I, P, P, P, P, I, I, I, I, I, I, I, P]
    ms_gdr_prepare = [P, I, I, I, I, P, I, P, P, P, LL, LL, P, P, P, P, P, I, I, I, I, I, F, P]
    ms_gdr_conv_update = [P, I, I, I, P, LL, LL, P, P, P, I, I, P]
    ms_gdr_scan = [P, P, P, LL, P, P, P, P, I, I, I, I, I, I, P]
    ms_moe_route_scored = [P, P, I, I, I, I, F, P, P, I, P]
    ms_gated_act_mul = [P, I, P, I, I, I, I, P]
    ms_head_norm_store = [P, I, P, P, P, F, F, I, I, P, P, P, I, I, I, P, P, P, P, I, I, I, I, I, I, I, I, P]
    ms_attention_wide_scored = [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, F, P, I, I, I, P]
    ms_attention_wide_mma_scored = [P, P, P, P, P, P, P, P, I, I, P, P, I, I, I, I, I, I, I, I, I, F, I, P, F, P, I, I, P]
    ms_gla_decay = [P, I, P, I, P, I, F, P, I, I, P]
    ms_gla_scan = [P, I, I, I, I, P, F, P, P, P, P, P, I, I, I, I, I, P]
    ms_gla_output = [P, I, P, I, P, F, P, I, I, I, I, P]
    ms_moe_route = [P, P, I, I, P, P, I, P]
    ms_moe_gate_up_pairs = [P, P, P, P, P, P, I, I, I, I, I, I, I, P]
    ms_moe_down_pairs = [P, P, P, P, P, P, I, I, I, I, I, I, P]
    ms_moe_grouped = [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P]
    ms_attention_wide = [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P]
    ms_attention_wide_mma = [P, P, P, P, P, P, P, P, I, I, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P]
    ms_rope_kv_store = [P, I, I, P, P, P, P, I, I, P, I, I, P, P, P, I, I, I, I, I, I, P]
    ms_attention_generic = [P, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    ms_gemm_f32 = [P, I, P, P, P, I, I, I, I, P]
    ms_attention_decode = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    ms_gemm_small_m_plan = [I, I, I, I, I, I, P]
    ms_attention_decode_cluster = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, I, I, P, LL, P, I, P]
    ms_attention_decode_cluster_sinks = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, I, I, P, LL, P, I, P, P]
    ms_attention_decode_cluster_rope = [P, I, P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, I, I, P, LL, P, I, P]
    ms_attention_prefill_tc = [P, P, P, P, I, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, LL, P, LL, P]
    ms_attention_prefill_tc_plan = [I, I, I, I, I, I, I, P]
    ms_attention_prefill_tc_sinks = [P, P, P, P, I, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, LL, P, LL, P, P]
    ms_attention_prefill = [P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P]
    ms_gemm_small_m = [P, I, P, P, I, I, I, I, I, I, P]
    ms_gemm_small_m_silu_mul = [P, I, P, P, P, I, I, I, I, I, P]
    ms_gemm_small_m_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_small_m_scaled = [P, I, P, I, F, P, P, P, I, I, I, I, I, P]
    ms_gemm_tc = [P, I, P, P, I, I, I, I, I, P]
    ms_gemm_tc_silu_mul = [P, I, P, P, I, I, I, I, P]
    ms_gemm_rows_tc = [P, I, P, P, I, I, I, I, I, I, P]
    ms_gemm_rows_tc_silu_mul = [P, I, P, P, P, I, I, I, I, I, P]
    ms_gemm_rows_tc_scaled = [P, I, P, I, F, P, P, P, I, I, I, I, I, P]
    ms_gemm_rows_tc_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_pair_tc = [P, I, P, P, I, I, I, I, P, I, F, I, P]
    ms_gemm_pair_tc_silu_mul = [P, I, P, P, I, I, I, I, P, I, F, I, P]
    ms_gemm_pair_tc_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_tc_wait_probe = [I, P]
    ms_attention_tc_wait_probe = [I, P]
    ms_take_sampled_tokens = [P, P, P, I, I, P]
    ms_apply_logit_offsets = [P, I, I, P, P, P, P]
    ms_sample = [P, I, I, P, P, P, P, P, P, P]
    ms_top_logprobs = [P, I, I, P, P, P, P, P]


_launches = 0


def launches() -> int:
    """How many of this library's kernels were launched so far in this process."""
    return _launches


def count_launches(n: int) -> None:
    """Adds launches that did not pass through the wrappers: kernels replayed from a captured graph."""
    global _launches
    _launches += n


def _check(code: int, name: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{name}: {lib().ms_last_error().decode()}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle (the capturing stream while a graph is captured).  Asked for with every launch, so
    through torch's raw getter where it exists: `torch.cuda.current_stream()` builds a Python object each time."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("a tensor on the CPU was given to a CUDA kernel; there is no CPU path")
    return c_void_p(t.data_ptr())


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ---------------------------------------------------------------------------


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, :] = table[ids[r], :] widened to float32.  table [V, d]; ids int32 [R]; out float32 [R, d]."""
    rows, d = out.shape
    _need(out.dtype == torch.float32 and ids.dtype == torch.int32 and ids.numel() >= rows, "embed_gather: bad arguments")
    _need(table.is_contiguous() and out.is_contiguous() and table.shape[1] == d, "embed_gather: bad layout")
    _check(
        lib().ms_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), rows, d, table.shape[0], _stream()),
        "embed_gather",
    )
    return out


def take_sampled_tokens(ids: torch.Tensor, from_rows: torch.Tensor, sampled: torch.Tensor) -> None:
    """ids[i] = sampled[from_rows[i]] where from_rows[i] >= 0 (all int32, on the device)."""
    _need(ids.dtype == torch.int32 and from_rows.dtype == torch.int32 and sampled.dtype == torch.int32 and
          from_rows.numel() >= ids.numel(), "take_sampled_tokens: bad arguments")
    _check(lib().ms_take_sampled_tokens(_ptr(ids), _ptr(from_rows), _ptr(sampled), ids.numel(), sampled.numel(), _stream()),
           "take_sampled_tokens")


def add_rmsnorm(
    residual: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    rows: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out = rmsnorm(residual + delta) * weight; without `rows` the sum is written back to `residual`.

    residual float32 [T, d]; delta [T, d] float32 or bfloat16 or None; weight float32 [d];
    out [n_out, d]; rows int32 [n_out] picks input rows (then nothing is written back).
    """
    d = residual.shape[1]
    n_out = out.shape[0]
    _need(residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d, "add_rmsnorm: bad dtypes")
    _need(residual.is_contiguous() and out.is_contiguous() and out.shape[1] == d, "add_rmsnorm: bad layout")
    if delta is not None:
        _need(delta.shape[1] == d and delta.is_contiguous() and delta.shape[0] >= residual.shape[0], "add_rmsnorm: bad delta")
    if rows is None:
        _need(n_out == residual.shape[0], "add_rmsnorm: out must have the residual's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_out, "add_rmsnorm: bad row list")
    _check(
        lib().ms_add_rmsnorm(
            _ptr(residual),
            _ptr(delta),
            _code(delta) if delta is not None else F32,
            _ptr(weight),
            _ptr(out),
            _code(out),
            _ptr(rows),
            n_out,
            d,
            float(eps),
            _stream(),
        ),
        "add_rmsnorm",
    )
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[r, c] += bias[c]: out [rows, n] float32 or bfloat16 (unit column stride), bias float32 [n]."""
    rows, n = out.shape
    _need(out.stride(1) == 1 and bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n, "add_bias: bad arguments")
    _check(lib().ms_add_bias(_ptr(out), _code(out), _ptr(bias), rows, n, out.stride(0), _stream()), "add_bias")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c].  gate_up [R, 2*inter], out [R, inter]."""
    rows, inter = out.shape
    _need(gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype, "silu_mul: bad shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous(), "silu_mul: bad layout")
    _check(lib().ms_silu_mul(_ptr(gate_up), _ptr(out), _code(out), rows, inter, _stream()), "silu_mul")
    return out


def rope_kv_store(
    qkv: torch.Tensor,
    bias: Optional[torch.Tensor],
    positions: torch.Tensor,
    seq_of_token: torch.Tensor,
    block_table: Optional[torch.Tensor],
    cos_sin: Optional[torch.Tensor],
    rotary_dim: int,
    interleaved: bool,
    q_out: torch.Tensor,
    k_pages: Optional[torch.Tensor],
    v_pages: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
) -> torch.Tensor:
    """Bias, rotary encoding of q and k, and the write of k, v into their pages.

    qkv [T, >= (Hq + 2*Hkv)*hd]; q_out [T, Hq*hd]; pages [num_pages, Hkv, page, hd];
    block_table int32 [S, max_pages]; cos_sin float32 [positions, rotary_dim/2, 2].
    With num_kv_heads == 0 only q is encoded.
    """
    tokens = q_out.shape[0]
    _need(qkv.stride(1) == 1 and q_out.is_contiguous() and q_out.dtype == qkv.dtype, "rope_kv_store: bad layout")
    _need(positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32, "rope_kv_store: index arrays must be int32")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() >= (num_heads + 2 * num_kv_heads) * head_dim),
          "rope_kv_store: bias must be float32 over q|k|v")
    if num_kv_heads:
        _need(k_pages is not None and k_pages.is_contiguous() and v_pages.is_contiguous(), "rope_kv_store: bad pages")
        _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "rope_kv_store: bad page shape")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "rope_kv_store: bad block table")
        num_pages, page_size, max_pages = k_pages.shape[0], k_pages.shape[2], block_table.shape[1]
        cache_code = _code(k_pages)
    else:
        num_pages = page_size = max_pages = 0
        cache_code = _code(qkv)
    if rotary_dim:
        _need(cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous(), "rope_kv_store: bad table")
        _need(cos_sin.shape[1] * 2 == rotary_dim, "rope_kv_store: table width does not match the rotary size")
    _check(
        lib().ms_rope_kv_store(
            _ptr(qkv), _code(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(seq_of_token), _ptr(block_table),
            max_pages, num_pages, _ptr(cos_sin), rotary_dim, int(interleaved), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
            cache_code, tokens, num_heads, num_kv_heads, head_dim, page_size, _stream(),
        ),
        "rope_kv_store",
    )
    return q_out


def attention_generic(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    positions: torch.Tensor,
    seq_of_token: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: Optional[int],
    scale: float,
    share_rows: bool = False,
) -> torch.Tensor:
    """The exact paged attention kernel.  q, out [T, Hq*hd]; pages [num_pages, Hkv, page, hd].  `share_rows`: rows that
    follow one another in a sequence (portions of prompts) share the tiles of keys they read, eight rows a block; the
    results are the same bits either way.  (A negative `share_rows`, for measurements: the float32 decoding form with
    that many heads of a group to a block.)"""
    tokens = q.shape[0]
    _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype, "attention: bad layout")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype, "attention: bad pages")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")
    _check(
        lib().ms_attention_generic(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _code(q), _code(k_pages), _ptr(positions),
            _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(share_rows), _stream(),
        ),
        "attention_generic",
    )
    return out


def attention_decode_supports(head_dim: int, groups: int) -> bool:
    return bool(lib().ms_attention_decode_supports(int(head_dim), int(groups)))


def attention_decode_scratch_words(tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, num_splits: int) -> int:
    """4-byte words of scratch for `num_splits` > 1: partial results, and one counter per (row, kv head)
    at the end, which must be zero before the first launch and is left zero by every launch."""
    return tokens * num_heads * num_splits * (head_dim + 2) + tokens * num_kv_heads if num_splits > 1 else 0


def attention_decode(q, k_pages, v_pages, out, scratch, positions, slot_of_token, block_table, num_heads, num_kv_heads,
                     head_dim, window, scale, num_splits, rows=None, num_rows=None):
    """Tensor-core paged attention for rows that are each attended on their own (decoding), bfloat16.
    `scratch` is float32 with at least attention_decode_scratch_words(...) elements whose tail (the
    counters) is zero (None for one split).
    `rows` (int32) lists the rows to attend, `num_rows` of them; by default every row of q."""
    tokens = q.shape[0] if rows is None else int(num_rows)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode: bad row list")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_decode: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode: bad block table")
    need = attention_decode_scratch_words(tokens, num_heads, num_kv_heads, head_dim, num_splits)
    _need(need == 0 or (scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need),
          "attention_decode: scratch is too small")
    _check(
        lib().ms_attention_decode(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(rows), _ptr(positions),
            _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(num_splits), _stream(),
        ),
        "attention_decode",
    )
    return out


def attention_decode_cluster_max_stages(head_dim: int) -> int:
    return int(lib().ms_attention_decode_cluster_max_stages(int(head_dim)))


def attention_decode_cluster_blocks_per_sm(head_dim: int, stages: int, warps: int = 4) -> int:
    """How many blocks of the kernel with `stages` tiles each an SM holds at once."""
    return int(lib().ms_attention_decode_cluster_blocks_per_sm(int(head_dim), int(stages), int(warps)))


def attention_decode_cluster_scratch_words(tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, parts: int) -> int:
    """float32 words of scratch for `parts` > 1 clusters per (row, kv head); beside them, tokens * num_kv_heads int32
    counters that are zero before the first launch."""
    fn = lib().ms_attention_decode_cluster_scratch_words
    fn.restype = c_longlong
    return int(fn(int(tokens), int(num_heads), int(num_kv_heads), int(head_dim), int(parts)))


def _outer_args(name, tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters):
    if parts <= 1:
        return 1, None, 0, None, 0
    need = attention_decode_cluster_scratch_words(tokens, num_heads, num_kv_heads, head_dim, parts)
    _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
          f"{name}: {parts} clusters a row need {need} float32 words of scratch")
    _need(counters is not None and counters.dtype == torch.int32 and counters.is_contiguous() and counters.numel() >= tokens * num_kv_heads,
          f"{name}: {parts} clusters a row need {tokens * num_kv_heads} int32 counters")
    return int(parts), _ptr(scratch), scratch.numel(), _ptr(counters), counters.numel()


def attention_decode_cluster(q, k_pages, v_pages, out, positions, slot_of_token, block_table, num_heads, num_kv_heads,
                             head_dim, window, scale, num_splits, stages, rows=None, num_rows=None, warps=4, keys_per_warp=0,
                             parts=1, scratch=None, counters=None, sinks=None):
    """As attention_decode, with the splits of a row held by one thread-block cluster (1, 2, 4 or 8) and merged in
    shared memory: no scratch.  Keys and values of earlier positions are requested before the kernel waits for its
    predecessor in the stream.  `stages`: tiles of 64 keys a block holds at once.  `parts` > 1 (few rows with long
    contexts): a row's keys go to that many clusters, which leave their sums in `scratch`; the one that ends last
    merges them in order (`counters`: int32 zeros, left zero).  `sinks` (float32, one per head): exp(sink) joins every
    row's softmax denominator and has no value."""
    tokens = q.shape[0] if rows is None else int(num_rows)
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads), "attention_decode_cluster: bad sinks")
    outer = _outer_args("attention_decode_cluster", tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode_cluster: bad row list")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_decode_cluster: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode_cluster: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode_cluster: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode_cluster: bad block table")
    _check(
        lib().ms_attention_decode_cluster_sinks(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(rows), _ptr(positions), _ptr(slot_of_token),
            _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads, num_kv_heads, head_dim,
            k_pages.shape[2], int(window or 0), float(scale), int(num_splits), int(stages), int(warps), int(keys_per_warp), *outer,
            _ptr(sinks), _stream(),
        ),
        "attention_decode_cluster",
    )
    return out


def attention_decode_cluster_rope(qkv, bias, cos_sin, store, k_pages, v_pages, out, positions, slot_of_token, block_table,
                                  num_heads, num_kv_heads, head_dim, window, scale, num_splits, stages, rows=None,
                                  num_rows=None, warps=4, keys_per_warp=0, parts=1, scratch=None, counters=None):
    """rope_kv_store and attention_decode_cluster in one kernel, for rows that are alone in their sequences: reads
    rows of q|k|v (k and v only if `store`) as the projection left them, adds the bias, rotates q and k (full rotary,
    pairs j and j + head_dim/2, table [positions, head_dim/2, 2]), writes k and v into the cache, and attends."""
    tokens = qkv.shape[0] if rows is None else int(num_rows)
    outer = _outer_args("attention_decode_cluster_rope", tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode_cluster_rope: bad row list")
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and
          v_pages.dtype == torch.bfloat16, "attention_decode_cluster_rope: bfloat16 only")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode_cluster_rope: bad layout")
    width = (num_heads + (2 * num_kv_heads if store else 0)) * head_dim
    _need(qkv.shape[1] >= width, "attention_decode_cluster_rope: rows are narrower than q|k|v")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() >= width),
          "attention_decode_cluster_rope: bad bias")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == head_dim,
          "attention_decode_cluster_rope: the table must be [positions, head_dim/2, 2] float32")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode_cluster_rope: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode_cluster_rope: bad block table")
    _check(
        lib().ms_attention_decode_cluster_rope(
            _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(cos_sin), 1 if store else 0, _ptr(k_pages), _ptr(v_pages), _ptr(out),
            _ptr(rows), _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0],
            tokens, num_heads, num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(num_splits),
            int(stages), int(warps), int(keys_per_warp), *outer, _stream(),
        ),
        "attention_decode_cluster_rope",
    )
    return out


def attention_prefill_supports(head_dim: int) -> bool:
    return bool(lib().ms_attention_prefill_supports(int(head_dim)))


def attention_prefill(q, k_pages, v_pages, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table,
                      num_heads, num_kv_heads, head_dim, window, scale):
    """Tensor-core paged causal attention for tiles of up to 64 consecutive rows of one sequence, bfloat16."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_prefill: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_prefill: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_prefill: bad block table")
    _need(tile_row0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and min(tile_row0.numel(), tile_rows.numel()) >= num_tiles,
          "attention_prefill: bad tile lists")
    _check(
        lib().ms_attention_prefill(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tile_row0), _ptr(tile_rows), int(num_tiles),
            _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), _stream(),
        ),
        "attention_prefill",
    )
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias), all float32, on the CUDA cores."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: all operands must be float32")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_f32: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_f32: bad output shape")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == n), "gemm_f32: bad bias")
    _check(
        lib().ms_gemm_f32(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), out.stride(0), m, n, k, _stream()),
        "gemm_f32",
    )
    return out


SMALL_M = 16  # up to this many rows the weight-streaming kernel is used instead of the library
SMALL_M_MAX_WEIGHT_BYTES = 64 << 20  # a larger matrix (the vocabulary head) streams faster through the library
_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def gemm_small_m_supports(m: int, n: int, k: int) -> bool:
    """Whether the kernel covers the sizes (M up to 64, K in steps of 8)."""
    return 1 <= m <= 64 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_small_m_preferred(m: int, n: int, k: int) -> bool:
    """Whether the engine uses it: measured on B200 against the library at the decoder's sizes."""
    return gemm_small_m_supports(m, n, k) and m <= SMALL_M and 2 * n * k <= SMALL_M_MAX_WEIGHT_BYTES


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64: bfloat16 operands, bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_small_m: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_small_m: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_small_m: bad output shape")
    _check(
        lib().ms_gemm_small_m(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, sm_count(),
                              _stream()),
        "gemm_small_m",
    )
    return out


def gemm_small_m_silu_mul(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) for M <= 64, all bfloat16, in one kernel."""
    m, k = x.shape
    i = w_gate.shape[0]
    _need(x.dtype == w_gate.dtype == w_up.dtype == out.dtype == torch.bfloat16, "gemm_small_m_silu_mul: bfloat16 only")
    _need(w_gate.is_contiguous() and w_up.is_contiguous() and tuple(w_up.shape) == (i, k) and w_gate.shape[1] == k,
          "gemm_small_m_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_small_m_silu_mul: bad layout")
    _check(
        lib().ms_gemm_small_m_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(out), out.stride(0), m, i, k,
                                       sm_count(), _stream()),
        "gemm_small_m_silu_mul",
    )
    return out


def gemm_small_m_plan(m: int, n: int, k: int, gated: bool = False, residual: bool = False, sms: Optional[int] = None) -> dict:
    """How the few-row product of m rows with n outputs over k is spread over a GPU of `sms` SMs (this one's by default):
    host arithmetic only."""
    plan = (c_int * 7)()
    _check(lib().ms_gemm_small_m_plan(int(m), int(n), int(k), 1 if gated else 0, 1 if residual else 0,
                                      int(sms) if sms else sm_count(), plan), "gemm_small_m_plan")
    names = ("warps", "row_blocks", "cluster", "staged_chunks", "held_chunks", "activation_stride", "shared_bytes")
    return dict(zip(names, (int(v) for v in plan)))


def gemm_small_m_stats_blocks(n: int) -> int:
    """How many blocks of 16 columns `gemm_small_m_resadd` leaves sums of squares for."""
    return (n + 15) // 16


def gemm_small_m_resadd(x, w, residual, stats_out, copy_out=None):
    """residual[M, N] += x[M, K] . w[N, K]^T in place (float32); stats_out[m][b] = sum of squares of the new
    residual's row m over its b-th block of 16 columns; copy_out (optional, bfloat16 [M, N]) = the new residual
    rounded.  M <= 16."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_small_m_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_small_m_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_small_m_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_small_m_stats_blocks(n),
          "gemm_small_m_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_small_m_resadd: the copy must be bfloat16 [rows, N]")
    _check(
        lib().ms_gemm_small_m_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                     _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                     _stream()),
        "gemm_small_m_resadd",
    )
    return residual


def gemm_small_m_scaled(x, stats, stats_blocks, eps, w, w_up, out):
    """out = (x . w^T) / rms(row), or silu(. w^T / rms) * (. w_up^T / rms) when w_up is given: x is the residual
    rounded to bfloat16 [M, K] (the copy gemm_small_m_resadd leaves), `stats` [M, stats_blocks] its sums of squares;
    the RMS norm for matrices that have the norm's weight folded into their columns.  M <= 16."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and stats.dtype == torch.float32 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "gemm_small_m_scaled: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k, "gemm_small_m_scaled: bad weights")
    _need(w_up is None or (w_up.dtype == torch.bfloat16 and w_up.is_contiguous() and tuple(w_up.shape) == (n, k)),
          "gemm_small_m_scaled: bad up weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n), "gemm_small_m_scaled: bad layout")
    _need(stats.is_contiguous() and stats.numel() >= m * stats_blocks, "gemm_small_m_scaled: bad stats buffer")
    _check(
        lib().ms_gemm_small_m_scaled(_ptr(x), x.stride(0), _ptr(stats), int(stats_blocks), float(eps), _ptr(w), _ptr(w_up),
                                     _ptr(out), out.stride(0), m, n, k, sm_count(), _stream()),
        "gemm_small_m_scaled",
    )
    return out


def gemm_tc_supports(m: int, n: int, k: int) -> bool:
    return m >= 1 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T on tcgen05 tensor cores with TMA-fed operands; bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_tc: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_tc: bad output shape")
    _check(lib().ms_gemm_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, _stream()), "gemm_tc")
    return out


def gemm_tc_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w[:I]^T) * (x . w[I:]^T) in one tcgen05 kernel; w_gate_up is [2I, K], gate rows first."""
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    _need(x.dtype == w_gate_up.dtype == out.dtype == torch.bfloat16, "gemm_tc_silu_mul: bfloat16 only")
    _need(w_gate_up.is_contiguous() and w_gate_up.shape[1] == k and w_gate_up.shape[0] == 2 * i, "gemm_tc_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_tc_silu_mul: bad layout")
    _check(lib().ms_gemm_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(out), out.stride(0), m, i, k, _stream()),
           "gemm_tc_silu_mul")
    return out


def gemm_rows_tc_supports(m: int, n: int, k: int) -> bool:
    """Up to 64 rows, K in steps of 8."""
    return 1 <= m <= 64 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_rows_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64 on tcgen05 tensor cores with the weights as the 128-row operand,
    streamed once through TMA stages; bfloat16 operands, bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_rows_tc: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_rows_tc: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_rows_tc: bad output shape")
    _check(lib().ms_gemm_rows_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, sm_count(), _stream()),
           "gemm_rows_tc")
    return out


def gemm_rows_tc_silu_mul(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) for M <= 64, all bfloat16, in one kernel."""
    m, k = x.shape
    i = w_gate.shape[0]
    _need(x.dtype == w_gate.dtype == w_up.dtype == out.dtype == torch.bfloat16, "gemm_rows_tc_silu_mul: bfloat16 only")
    _need(w_gate.is_contiguous() and w_up.is_contiguous() and tuple(w_up.shape) == (i, k) and w_gate.shape[1] == k,
          "gemm_rows_tc_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_rows_tc_silu_mul: bad layout")
    _check(lib().ms_gemm_rows_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(out), out.stride(0), m, i, k,
                                          sm_count(), _stream()), "gemm_rows_tc_silu_mul")
    return out


def gemm_rows_tc_resadd(x, w, residual, stats_out, copy_out=None):
    """As gemm_small_m_resadd, for up to 64 rows: residual += x . w^T (float32, in place), the sums of squares of the
    new residual per row and block of 16 columns, and optionally its bfloat16 copy."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_rows_tc_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_rows_tc_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_rows_tc_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_small_m_stats_blocks(n),
          "gemm_rows_tc_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_rows_tc_resadd: the copy must be bfloat16 [rows, N]")
    _check(lib().ms_gemm_rows_tc_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                        _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                        _stream()), "gemm_rows_tc_resadd")
    return residual


def gemm_rows_tc_scaled(x, stats, stats_blocks, eps, w, w_up, out):
    """As gemm_small_m_scaled, for up to 64 rows: out = (x . w^T) / rms(row), or the gated form with w_up."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and stats.dtype == torch.float32 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "gemm_rows_tc_scaled: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k, "gemm_rows_tc_scaled: bad weights")
    _need(w_up is None or (w_up.dtype == torch.bfloat16 and w_up.is_contiguous() and tuple(w_up.shape) == (n, k)),
          "gemm_rows_tc_scaled: bad up weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n), "gemm_rows_tc_scaled: bad layout")
    _need(stats.is_contiguous() and stats.numel() >= m * stats_blocks, "gemm_rows_tc_scaled: bad stats buffer")
    _check(lib().ms_gemm_rows_tc_scaled(_ptr(x), x.stride(0), _ptr(stats), int(stats_blocks), float(eps), _ptr(w), _ptr(w_up),
                                        _ptr(out), out.stride(0), m, n, k, sm_count(), _stream()), "gemm_rows_tc_scaled")
    return out


def gemm_pair_tc(x, w, out, stats=None, stats_blocks=0, eps=0.0):
    """out[M, N] = x[M, K] . w[N, K]^T for many rows on the tcgen05 tensor cores (a pair of SMs per tile, resident
    blocks that go through their tiles, two accumulators in tensor memory), all bfloat16.  With `stats` ([M, stats_blocks] sums of
    squares of the rows x was rounded from) every output row is divided by that row's rms: the RMS norm for a matrix
    with the norm's weight folded into its columns."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "gemm_pair_tc: bfloat16 only")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n),
          "gemm_pair_tc: bad layout")
    _need(stats is None or (stats.dtype == torch.float32 and stats.is_contiguous() and stats.numel() >= m * stats_blocks >= m),
          "gemm_pair_tc: bad stats buffer")
    _check(lib().ms_gemm_pair_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), out.stride(0), m, n, k, _ptr(stats), int(stats_blocks),
                                   float(eps), sm_count(), _stream()), "gemm_pair_tc")
    return out


# From where the gated product with the gating in its epilogue beats the library's product followed by the gating
# kernel (measured on B200 at K = 896, 1,536, 2,048 and 3,584, 256 to 4,152 rows: from 1,024 rows on by 6 to 17 %,
# at K = 896 only from 2,048 rows on; below 1,024 rows the library wins).
PAIR_TC_SILU_MIN_ROWS = 1024
PAIR_TC_SILU_MIN_ROWS_NARROW = 2048  # for K below 1,024


def gemm_pair_tc_silu_preferred(m: int, i: int, k: int) -> bool:
    return m >= (PAIR_TC_SILU_MIN_ROWS if k >= 1024 else PAIR_TC_SILU_MIN_ROWS_NARROW) and i % 8 == 0 and k % 8 == 0


def gemm_pair_tc_silu_mul(x, w_gate_up, out, stats=None, stats_blocks=0, eps=0.0):
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) with w_gate_up = [gate rows; up rows] ([2I, K]); row scaling as in
    gemm_pair_tc."""
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "gemm_pair_tc_silu_mul: bfloat16 only")
    _need(w_gate_up.is_contiguous() and w_gate_up.shape[1] == k and w_gate_up.shape[0] == 2 * i and x.stride(1) == 1 and
          out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_pair_tc_silu_mul: bad layout")
    _need(stats is None or (stats.dtype == torch.float32 and stats.is_contiguous() and stats.numel() >= m * stats_blocks >= m),
          "gemm_pair_tc_silu_mul: bad stats buffer")
    _check(lib().ms_gemm_pair_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(out), out.stride(0), m, i, k, _ptr(stats),
                                            int(stats_blocks), float(eps), sm_count(), _stream()), "gemm_pair_tc_silu_mul")
    return out


def gemm_pair_tc_stats_blocks(m: int, n: int) -> int:
    """How many sums of squares per row `gemm_pair_tc_resadd` leaves for a residual of [m, n] (one per tile of columns)."""
    return int(lib().ms_gemm_pair_tc_stats_blocks(int(m), int(n), sm_count()))


def gemm_pair_tc_resadd(x, w, residual, stats_out, copy_out=None):
    """residual[M, N] += x[M, K] . w[N, K]^T in place (float32), the sums of squares of the new residual per row and
    tile of columns (`gemm_pair_tc_stats_blocks` of them a row; a consumer adds up all of a row's), and optionally its
    bfloat16 copy; any number of rows."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_pair_tc_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_pair_tc_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_pair_tc_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_pair_tc_stats_blocks(m, n),
          "gemm_pair_tc_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_pair_tc_resadd: the copy must be bfloat16 [rows, N]")
    _check(lib().ms_gemm_pair_tc_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                          _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                          _stream()), "gemm_pair_tc_resadd")
    return residual


def gemm_tc_status(reset: bool = True) -> int:
    """0, or which bounded wait of a tcgen05 kernel gave up (products: 1 producer, 2 issuer, 3 epilogue, 21-23 the same of the
    resident-block product; attention: 11 producer, 12-14 and 16 issuer, 15 softmax threads).  Synchronizes."""
    codes = tc_status_codes(reset)
    return codes[0] or codes[1]


def tc_status_codes(reset: bool = True):
    """(code of the tcgen05 products, code of the tcgen05 attention): both are read, and cleared with `reset`,
    whichever of them is set.  Synchronizes."""
    lib()  # (kernels that are not in the loaded library cannot have given up a wait)
    gemm = int(_lib.ms_gemm_tc_status(1 if reset else 0)) if has("ms_gemm_tc_status") else 0
    attention = int(_lib.ms_attention_tc_status(1 if reset else 0)) if has("ms_attention_tc_status") else 0
    return gemm, attention


def tc_wait_probe(kernel: str, polls: int = 1000) -> None:
    """Launches one thread that waits `polls` polls on a barrier nothing arrives on, through the bounded-wait helper
    of the tcgen05 products (`kernel="gemm"`, leaves code 9) or of the tcgen05 attention (`"attention"`, code 19):
    the way to see the give-up path run (error word set, kernel returns, context usable) without a hang."""
    _need(kernel in ("gemm", "attention"), "tc_wait_probe: kernel is 'gemm' or 'attention'")
    fn = lib().ms_gemm_tc_wait_probe if kernel == "gemm" else lib().ms_attention_tc_wait_probe
    _check(fn(int(polls), _stream()), "tc_wait_probe")


def attention_prefill_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().ms_attention_prefill_tc_supports(int(head_dim), int(page_size)))


def attention_prefill_tc_plan(num_tiles: int, num_heads: int, num_kv_heads: int, head_dim: int, max_keys: int,
                              key_tiles: int = 0):
    """(splits, alone, run_tiles): into how many runs the kernel should cut an item's key tiles so that the launch fills
    the GPU (1 to 4), whether, at head size 128, every block should take one head instead of two of a group, and (if
    not 0) the most key tiles of a run, so that only longer items are cut.
    `key_tiles`: the tiles of 128 keys that the launch's tiles of rows see, in all (0: every tile sees `max_keys`)."""
    plan = (ctypes.c_int * 3)()
    lib().ms_attention_prefill_tc_plan(int(num_tiles), int(num_heads), int(num_kv_heads), int(head_dim), int(max_keys),
                                       int(key_tiles), sm_count(), plan)
    return int(plan[0]), bool(plan[1]), int(plan[2])


def attention_prefill_tc_scratch_words(num_tiles: int, num_heads: int, head_dim: int, splits: int) -> int:
    """float32 words of scratch memory for `splits` > 1 (beside num_tiles * num_heads int32 counters, which must be zero
    before the first launch and are left zero by every launch)."""
    fn = lib().ms_attention_prefill_tc_scratch_words
    fn.restype = c_longlong
    return int(fn(int(num_tiles), int(num_heads), int(head_dim), int(splits)))


def attention_prefill_tc(q, k_pages, v_pages, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table,
                         num_heads, num_kv_heads, head_dim, window, scale, splits=1, scratch=None, counters=None, alone=False,
                         run_tiles=0, sinks=None):
    """Paged causal attention for tiles of up to 128 consecutive rows of one sequence on tcgen05 tensor cores
    (TMA-fed, scores in tensor memory and taken into registers a row per thread, probabilities back into tensor
    memory, outputs accumulated there over all key tiles).  Head sizes 64 (one head per block) and 128 (two heads of a
    group per block, which share the keys and values), page sizes 8, 16, 32, ...  With `splits` > 1 the key tiles of
    every (tile, head) go to that many blocks, which meet in `scratch` (float32) and count themselves in `counters`
    (int32, num_tiles * num_heads of them, all zero before and after).  `alone` (head size 128): one head per block.
    `run_tiles` > 0: only items with more key tiles are cut, into runs of at most that many.  `sinks` (float32, one per
    head): exp(sink) joins every row's softmax denominator and has no value."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_prefill_tc: bfloat16 only")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads), "attention_prefill_tc: bad sinks")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_prefill_tc: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_prefill_tc: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_prefill_tc: bad block table")
    _need(tile_row0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and min(tile_row0.numel(), tile_rows.numel()) >= num_tiles,
          "attention_prefill_tc: bad tile lists")
    _need(scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()), "attention_prefill_tc: scratch must be float32")
    _need(counters is None or (counters.dtype == torch.int32 and counters.is_contiguous()), "attention_prefill_tc: counters must be int32")
    _check(
        lib().ms_attention_prefill_tc_sinks(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), q.shape[0], _ptr(tile_row0), _ptr(tile_rows), int(num_tiles),
            _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(splits), 1 if alone else 0, int(run_tiles), _ptr(scratch),
            scratch.numel() if scratch is not None else 0, _ptr(counters), counters.numel() if counters is not None else 0,
            _ptr(sinks), _stream(),
        ),
        "attention_prefill_tc",
    )
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out = x . w^T (+ bias, float32 [n]).  float32 goes to the CUDA-core kernel.  bfloat16 with few rows
    (decoding) goes to the weight-streaming tensor-core kernel; with many rows it goes to the
    library matrix product (cuBLAS through torch), where the reference too calls its library
    (hipBLAS GemmEx, crates/mach-model/src/kernels.rs:6416-6455 of gqf2008/machserve); a bias is then
    added by a kernel of its own (the built-in attention adds its bias inside its rotary kernel instead)."""
    if x.dtype == torch.float32:
        return gemm_f32(x, w, bias, out)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16 or float32")
    if gemm_small_m_preferred(x.shape[0], w.shape[0], x.shape[1]) and x.stride(0) % 8 == 0:
        gemm_small_m(x, w, out)
    elif out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return add_bias(out, bias) if bias is not None else out



# ------------------------------------------------------------------- parts of layers beyond the pre-norm decoder's


def _delta_args(delta):
    return (_ptr(delta), _code(delta) if delta is not None else F32)


def add_layernorm(residual, delta_a, delta_b, weight, bias, out, eps, rows=None, weight2=None, bias2=None, out2=None):
    """out = layernorm(residual + (delta_a + delta_b)) * weight + bias (mean and variance of the row, eps inside the
    root); without `rows` the sum is written back to `residual`.  With weight2, bias2 and out2 a second norm of the same
    rows is written beside the first (they share mean and variance).

    residual float32 [T, d]; deltas [T, d] float32 or bfloat16 or None; weights and biases float32 [d];
    out, out2 [n_out, d]; rows int32 [n_out] picks input rows (then nothing is written back)."""
    d = residual.shape[1]
    n_out = out.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous() and out.shape[1] == d,
          "add_layernorm: bad layout")
    for v in (weight, bias, weight2, bias2):
        _need(v is None or (v.dtype == torch.float32 and v.numel() == d and v.is_contiguous()), "add_layernorm: bad weight or bias")
    for dl in (delta_a, delta_b):
        _need(dl is None or (dl.shape[1] == d and dl.is_contiguous() and dl.shape[0] >= residual.shape[0]), "add_layernorm: bad delta")
    if out2 is not None:
        _need(weight2 is not None and bias2 is not None and out2.dtype == out.dtype and out2.is_contiguous()
              and tuple(out2.shape) == tuple(out.shape), "add_layernorm: bad second norm")
    if rows is None:
        _need(n_out == residual.shape[0], "add_layernorm: out must have the residual's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_out, "add_layernorm: bad row list")
    _check(lib().ms_add_layernorm(_ptr(residual), *_delta_args(delta_a), *_delta_args(delta_b), _ptr(weight), _ptr(bias), _ptr(out),
                                  _ptr(weight2), _ptr(bias2), _ptr(out2), _code(out), _ptr(rows), n_out, d, float(eps), _stream()),
           "add_layernorm")
    return out


def concat_streams(residual, delta_a, delta_b, other, out):
    """out[:, :d] = residual + (delta_a + delta_b), out[:, d:] = other: residual and other float32 [T, d], out [T, 2d]."""
    t, d = residual.shape
    _need(residual.dtype == torch.float32 and other.dtype == torch.float32 and residual.is_contiguous() and other.is_contiguous()
          and tuple(other.shape) == (t, d) and tuple(out.shape) == (t, 2 * d) and out.is_contiguous(), "concat_streams: bad arguments")
    for dl in (delta_a, delta_b):
        _need(dl is None or (dl.shape[1] == d and dl.is_contiguous() and dl.shape[0] >= t), "concat_streams: bad delta")
    _check(lib().ms_concat_streams(_ptr(residual), *_delta_args(delta_a), *_delta_args(delta_b), _ptr(other), _ptr(out), _code(out),
                                   t, d, _stream()), "concat_streams")
    return out


def glu_clamped(gate_up, out, limit: float, alpha: float, shift: float):
    """out = g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit);
    gate_up float32 [R, 2*inter] (gate first), out [R, inter] float32 or bfloat16."""
    rows, inter = out.shape
    _need(gate_up.shape[1] == 2 * inter and gate_up.dtype == torch.float32 and gate_up.is_contiguous() and out.is_contiguous(),
          "glu_clamped: bad arguments")
    _check(lib().ms_glu_clamped(_ptr(gate_up), _ptr(out), _code(out), rows, inter, float(limit), float(alpha), float(shift), _stream()),
           "glu_clamped")
    return out


def sigmoid_gate_mul(x, gate, out):
    """out = x * sigmoid(gate): x and gate float32 [R, n] with unit column stride (any row stride), out [R, n] contiguous."""
    rows, n = out.shape
    _need(x.dtype == torch.float32 and gate.dtype == torch.float32 and x.stride(1) == 1 and gate.stride(1) == 1
          and tuple(x.shape) == (rows, n) and tuple(gate.shape) == (rows, n) and out.is_contiguous(), "sigmoid_gate_mul: bad arguments")
    _check(lib().ms_sigmoid_gate_mul(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _ptr(out), _code(out), rows, n, _stream()),
           "sigmoid_gate_mul")
    return out


def qk_norm_store(proj, wq, wk, eps, coef, every, positions, slot_of_token, block_table, q_out, k_pages, v_pages,
                  groups: int, dk: int, dv: int, store: bool = True, q_half=None):
    """Unit-rms norm of the whole q and of the whole k projection with weights, query temperature
    1 + coef * ln(floor((p + 1) / every) + 1), q to q_out (float32), k and v into their pages.

    proj float32 [T, >= qw + groups*(dk + dv)] = [q | k | v]; wq [qw], wk [groups*dk] float32; q_out float32 [T, qw];
    k pages [pages, groups, page, dk], v pages [pages, groups, page, dv].  `q_half`: bfloat16 [T, qw], a rounded copy
    of the queries for a kernel that reads them so."""
    t, qw = q_out.shape
    _need(q_half is None or (q_half.dtype == torch.bfloat16 and q_half.is_contiguous() and tuple(q_half.shape) == (t, qw)),
          "qk_norm_store: bad bfloat16 copy of the queries")
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.dtype == torch.float32 and q_out.is_contiguous(),
          "qk_norm_store: bad layout")
    _need(wq.dtype == torch.float32 and wq.numel() == qw and wk.dtype == torch.float32 and wk.numel() == groups * dk,
          "qk_norm_store: bad norm weights")
    if store:
        _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype
              and tuple(k_pages.shape[1:]) == (groups, k_pages.shape[2], dk) and tuple(v_pages.shape[1:]) == (groups, k_pages.shape[2], dv),
              "qk_norm_store: bad pages")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "qk_norm_store: bad block table")
    _check(lib().ms_qk_norm_store(
        _ptr(proj), proj.stride(0), _ptr(wq), _ptr(wk), float(eps), float(coef), int(every), _ptr(positions), _ptr(slot_of_token),
        _ptr(block_table), block_table.shape[1] if store else 0, k_pages.shape[0] if store else 0, k_pages.shape[2] if store else 0,
        _ptr(q_out), _ptr(q_half), _ptr(k_pages if store else None), _ptr(v_pages if store else None), _code(k_pages) if store else F32,
        t, qw, groups, dk, dv, int(store), _stream()), "qk_norm_store")
    return q_out


def latent_encode(proj, kv_off, w_latent, eps, cos_sin, rot, positions, slot_of_token, block_table, q_wide, q_plain, pages,
                  heads: int, dn: int, dr: int, r: int, store: bool = True, queries=None, interleaved: bool = True):
    """Between the input product of a latent-attention mixer and its attention: the latent's unit-rms norm with weight
    and the rotated key part into the pages [pages, 1, page, r + dr]; the queries' rotated parts into q_wide[:, :, r:]
    (float32 [T, heads, r + dr]); their unrotated parts into q_plain [T, heads, dn] (the dtype their product reads).

    proj float32 [T, ld]: queries at column 0 head by head as [dn | dr], the down-projection [r | dr] at `kv_off`;
    cos_sin float32 [positions, rot/2, 2]: pairs of the first `rot` of the dr coordinates are turned, (2i, 2i + 1) when
    `interleaved`, else (i, i + rot/2).  `queries` (float32 [T, >= heads*(dn + dr)], unit column stride): the queries come from
    there instead of from column 0 of proj."""
    t = q_plain.shape[0]
    _need(queries is None or (queries.dtype == torch.float32 and queries.stride(1) == 1 and queries.shape[0] == t
                              and queries.shape[1] >= heads * (dn + dr)), "latent_encode: bad queries")
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and q_wide.dtype == torch.float32 and q_wide.is_contiguous()
          and q_plain.is_contiguous() and q_wide.numel() == t * heads * (r + dr) and q_plain.numel() == t * heads * dn,
          "latent_encode: bad layout")
    _need(w_latent.dtype == torch.float32 and w_latent.numel() == r, "latent_encode: bad norm weight")
    if rot:
        _need(cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot,
              "latent_encode: bad table of angles")
    if store:
        _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (1, pages.shape[2], r + dr), "latent_encode: bad pages")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "latent_encode: bad block table")
    _check(lib().ms_latent_encode(
        _ptr(proj), proj.stride(0), int(kv_off), _ptr(queries), queries.stride(0) if queries is not None else 0, _ptr(w_latent),
        float(eps), _ptr(cos_sin), int(rot), int(bool(interleaved)), cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slot_of_token), _ptr(block_table),
        block_table.shape[1] if store else 0, pages.shape[0] if store else 0, pages.shape[2] if store else 0, _ptr(q_wide),
        _ptr(q_plain), _code(q_plain), _ptr(pages if store else None), _code(pages) if store else _code(q_plain), t, heads, dn, dr, r,
        int(store), _stream()), "latent_encode")
    return q_wide


def attention_wide(q, k_pages, v_pages, out, sinks, positions, slot_of_token, block_table, num_heads: int, num_kv_heads: int,
                   dk: int, dv: int, window: Optional[int], scale: float, share_rows: bool = False, score: Optional["ScoreExtras"] = None):
    """The exact paged attention for keys and values of different widths, with an optional sink per head in the
    softmax's denominator.  q float32 [T, Hq*dk]; k pages [pages, Hkv, page, dk]; v pages [pages, Hkv, page, vw] of which
    the first dv columns are the values (the same array as the keys for a latent cache); out [T, Hq*dv] in the cache's
    dtype; sinks float32 [Hq] or None.  `share_rows` as in attention_generic: the same bits either way."""
    tokens = q.shape[0]
    _need(q.dtype == torch.float32 and q.is_contiguous() and out.is_contiguous() and out.dtype == k_pages.dtype
          and q.numel() == tokens * num_heads * dk and out.numel() == tokens * num_heads * dv, "attention_wide: bad layout")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype, "attention_wide: bad pages")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dk) and tuple(v_pages.shape[:3]) == tuple(k_pages.shape[:3])
          and v_pages.shape[3] >= dv, "attention_wide: bad page shapes")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads), "attention_wide: bad sinks")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_wide: bad block table")
    if score is not None:
        _check(lib().ms_attention_wide_scored(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _code(k_pages), _ptr(sinks), _ptr(positions), _ptr(slot_of_token),
            _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads, num_kv_heads, dk, dv, v_pages.shape[3],
            k_pages.shape[2], int(window or 0), float(scale), *score.args(num_heads), int(share_rows), _stream()), "attention_wide")
        return out
    _check(lib().ms_attention_wide(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _code(k_pages), _ptr(sinks), _ptr(positions), _ptr(slot_of_token),
        _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads, num_kv_heads, dk, dv, v_pages.shape[3],
        k_pages.shape[2], int(window or 0), float(scale), int(share_rows), _stream()), "attention_wide")
    return out


class ScoreExtras:
    """What the wide attention kernels may apply between the scaled score and the softmax, and a mask by chunks:
    `softcap` (score <- softcap * tanh(score / softcap); None or 0: none), `dist_bias` (float32 [heads, L]: the bias of head
    h at distance i - j is dist_bias[h, min(i - j, L - 1)], added after the cap and not scaled; None: none), `chunk` (position
    i sees the keys j <= i with j // chunk == i // chunk only; None or 0: every earlier key, or the window)."""

    def __init__(self, softcap=None, dist_bias: Optional[torch.Tensor] = None, chunk=None):
        self.softcap, self.dist_bias, self.chunk = float(softcap or 0.0), dist_bias, int(chunk or 0)
        _need(self.softcap >= 0.0 and self.chunk >= 0, "ScoreExtras: a negative cap or chunk")
        _need(dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and dist_bias.is_contiguous()
                                    and dist_bias.shape[1] > 0), "ScoreExtras: the distance bias must be float32 [heads, L]")

    def args(self, num_heads: int):
        b = self.dist_bias
        _need(b is None or b.shape[0] == num_heads, "ScoreExtras: the distance bias has another number of heads")
        return (c_float(self.softcap), _ptr(b), int(b.shape[1]) if b is not None else 0, self.chunk)


def attention_wide_mma_supports(dk: int, dv: int, vw: int, separate_v: bool) -> bool:
    """Whether the tensor-core form covers the widths (dk in steps of 16, dv and the value rows in steps of 8, dv <= 512,
    and a key tile that fits the shared memory)."""
    return bool(lib().ms_attention_wide_mma_supports(int(dk), int(dv), int(vw), int(separate_v)))


def attention_wide_mma_tile_rows(dv: int) -> int:
    """Rows of a portion that one block of the tensor-core form attends (64, 32 or 16, as the value columns leave registers)."""
    return int(lib().ms_attention_wide_mma_tile_rows(int(dv)))


def attention_wide_mma_scratch_words(items: int, dv: int, splits: int) -> int:
    """float32 words of scratch for `items` (decoding rows x key heads x chunks of 16 heads) cut into `splits` runs of keys."""
    fn = lib().ms_attention_wide_mma_scratch_words
    fn.restype = c_longlong
    fn.argtypes = [c_int, c_int, c_int]
    return int(fn(int(items), int(dv), int(splits)))


def attention_wide_mma(q, k_pages, v_pages, out, sinks, positions, slot_of_token, block_table, unit_row0, unit_rows, units: int,
                       heads: bool, num_heads: int, num_kv_heads: int, dk: int, dv: int, window: Optional[int], scale: float,
                       splits: int = 1, scratch: Optional[torch.Tensor] = None, score: Optional[ScoreExtras] = None):
    """attention_wide on the tensor cores (mma.sync, bfloat16 cache and output, float32 queries and softmax).
    heads False: `units` tiles of at most attention_wide_mma_tile_rows(dv) consecutive rows of one sequence, tile u = rows
    unit_row0[u] .. + unit_rows[u].
    heads True: `units` rows that are alone in their sequences (unit_row0[u], or u without a list; -1 for none); the query
    heads that share a key head fill the tensor core's rows, and a row's key tiles are cut into `splits` runs that meet in
    `scratch` (float32, attention_wide_mma_scratch_words).  v_pages may be k_pages itself (a latent cache)."""
    _need(q.dtype == torch.float32 and q.is_contiguous() and out.is_contiguous() and out.dtype == torch.bfloat16
          and k_pages.dtype == torch.bfloat16 and v_pages.dtype == torch.bfloat16, "attention_wide_mma: bad dtypes or layout")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dk)
          and tuple(v_pages.shape[:3]) == tuple(k_pages.shape[:3]) and v_pages.shape[3] >= dv, "attention_wide_mma: bad page shapes")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads), "attention_wide_mma: bad sinks")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_wide_mma: bad block table")
    for lst in (unit_row0, unit_rows):
        _need(lst is None or (lst.dtype == torch.int32 and lst.numel() >= units), "attention_wide_mma: bad unit lists")
    if splits > 1:
        groups = num_heads // num_kv_heads
        need = attention_wide_mma_scratch_words(units * num_kv_heads * (-(-groups // 16)), dv, splits)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need, "attention_wide_mma: scratch too small")
    if score is not None:
        _check(lib().ms_attention_wide_mma_scored(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(sinks), _ptr(positions), _ptr(slot_of_token), _ptr(block_table),
            block_table.shape[1], k_pages.shape[0], _ptr(unit_row0), _ptr(unit_rows), int(units), int(heads), num_heads, num_kv_heads,
            dk, dv, v_pages.shape[3], k_pages.shape[2], int(window or 0), float(scale), int(splits), _ptr(scratch),
            *score.args(num_heads), _stream()), "attention_wide_mma")
    else:
        _check(lib().ms_attention_wide_mma(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(sinks), _ptr(positions), _ptr(slot_of_token), _ptr(block_table),
            block_table.shape[1], k_pages.shape[0], _ptr(unit_row0), _ptr(unit_rows), int(units), int(heads), num_heads, num_kv_heads,
            dk, dv, v_pages.shape[3], k_pages.shape[2], int(window or 0), float(scale), int(splits), _ptr(scratch), _stream()),
            "attention_wide_mma")
    if splits > 1:
        count_launches(1)  # the merge of the splits
    return out


def linear_heads(x, w, out):
    """out[:, h, :] = x[:, h, :] . w[h]^T for every head h: x [T, H, a] and out [T, H, b] with unit stride along the last
    axis (any strides otherwise), w [H, b, a] contiguous.  float32 operands: one CUDA-core product per head (row results
    independent of the batch); bfloat16 operands: the library's batched product, out float32 or bfloat16."""
    t, heads, a = x.shape
    b = w.shape[1]
    _need(tuple(w.shape) == (heads, b, a) and w.is_contiguous() and tuple(out.shape) == (t, heads, b)
          and x.stride(2) == 1 and out.stride(2) == 1, "linear_heads: bad layout")
    if x.dtype == torch.float32:
        for h in range(heads):
            gemm_f32(x[:, h], w[h], None, out[:, h])
        return out
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_heads: operands must both be bfloat16 or float32")
    if out.dtype == torch.bfloat16:
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    else:
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32, out=out.transpose(0, 1))
    return out


# ------------------------------------------------- scaled embedding with positions, pair-adding RMS norm, gated activations


def embed_scaled_pos(table, ids, positions, pos_table, out, scale: float):
    """out[r, :] = table[ids[r], :] * scale + pos_table[positions[r], :] in float32.  table [V, d] float32 or bfloat16;
    pos_table float32 [P, d] or None; ids, positions int32 [R]; out float32 [R, d]."""
    rows, d = out.shape
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and table.shape[1] == d
          and ids.dtype == torch.int32 and positions.dtype == torch.int32 and ids.numel() >= rows and positions.numel() >= rows,
          "embed_scaled_pos: bad arguments")
    _need(pos_table is None or (pos_table.dtype == torch.float32 and pos_table.is_contiguous() and pos_table.shape[1] == d),
          "embed_scaled_pos: bad table of positions")
    _check(lib().ms_embed_scaled_pos(_ptr(table), _code(table), _ptr(ids), _ptr(positions), _ptr(pos_table), _ptr(out), rows, d,
                                     table.shape[0], pos_table.shape[0] if pos_table is not None else 0, float(scale), _stream()),
           "embed_scaled_pos")
    return out


def add_streams_rmsnorm(residual, delta_a, delta_b, first, vec, weight, out, eps: float = 0.0, rows=None, delta_scale: float = 1.0):
    """residual += delta_scale * (delta_a + delta_b) + first + vec (each may be None), then, with `weight`, out = residual / rms * weight.
    With `rows`, output row i comes from input row rows[i] and nothing is written back.  residual, first float32 [T, d];
    deltas [T, d] float32 or bfloat16; vec, weight float32 [d]; out [n_out, d] float32 or bfloat16 (None without a weight)."""
    t, d = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_streams_rmsnorm: bad stream")
    for dl in (delta_a, delta_b):
        _need(dl is None or (dl.shape[1] == d and dl.is_contiguous() and dl.shape[0] >= t), "add_streams_rmsnorm: bad delta")
    _need(first is None or (first.dtype == torch.float32 and first.is_contiguous() and first.shape[1] == d and first.shape[0] >= t),
          "add_streams_rmsnorm: bad second stream")
    for v in (vec, weight):
        _need(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == d), "add_streams_rmsnorm: bad vector")
    if weight is None:
        _need(out is None and rows is None, "add_streams_rmsnorm: an output without a weight")
        n_out = t
    else:
        _need(out is not None and out.is_contiguous() and out.shape[1] == d, "add_streams_rmsnorm: bad output")
        n_out = out.shape[0]
        if rows is None:
            _need(n_out == t, "add_streams_rmsnorm: out must have the stream's rows")
        else:
            _need(rows.dtype == torch.int32 and rows.numel() >= n_out, "add_streams_rmsnorm: bad row list")
    _check(lib().ms_add_streams_rmsnorm(_ptr(residual), *_delta_args(delta_a), *_delta_args(delta_b), _ptr(first), _ptr(vec), _ptr(weight),
                                        _ptr(out), _code(out) if out is not None else F32, _ptr(rows), n_out, d, float(eps), float(delta_scale),
                                        _stream()),
           "add_streams_rmsnorm")
    return out


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu": 2}  # "gelu": the exact form, 0.5 z (1 + erf(z / sqrt(2)))


def gated_act_mul(gate_up, out, activation: str):
    """out[r, c] = act(gate_up[r, c]) * gate_up[r, inter + c]; act "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))),
    in float32.  gate_up [R, 2*inter], out [R, inter], each float32 or bfloat16."""
    rows, inter = out.shape
    _need(activation in ACTIVATIONS, f"gated_act_mul: activation '{activation}' is not known ({', '.join(ACTIVATIONS)})")
    _need(tuple(gate_up.shape) == (rows, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous(), "gated_act_mul: bad layout")
    for r0 in range(0, rows, 65535):
        n = min(65535, rows - r0)
        _check(lib().ms_gated_act_mul(_ptr(gate_up[r0:]), _code(gate_up), _ptr(out[r0:]), _code(out), n, inter, ACTIVATIONS[activation],
                                      _stream()), "gated_act_mul")
    return out


def head_norm_store(proj, eps: float, positions, slot_of_token, block_table, q_out, k_pages, v_pages, num_heads: int, num_kv_heads: int,
                    dk: int, dv: int, v_off: Optional[int], norm: bool = True, wq=None, wk=None, store: bool = True, q_half=None,
                    bias=None, temp_coef: float = 0.0, temp_every: int = 1):
    """Every query head and every key head divided by its own root mean square over dk (eps inside the root; optional
    weights wq, wk float32 [dk]; `norm` False leaves them as they are); q to q_out (float32 [T, Hq*dk]) and, optionally, to
    a bfloat16 copy; the normed keys into k_pages; into v_pages the values at column `v_off` of the product, or, `v_off`
    None, the keys as they were projected (before the norm).  proj float32 [T, >= (Hq + Hkv)*dk (+ Hkv*dv)] = [q | k | v];
    `bias` (float32, one entry per column that is read, or None) is added to the product first.  With `temp_coef` c the
    query at position p is multiplied by 1 + c * ln(floor((p + 1) / temp_every) + 1)."""
    t = q_out.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.dtype == torch.float32 and q_out.is_contiguous()
          and q_out.numel() == t * num_heads * dk, "head_norm_store: bad layout")
    _need(q_half is None or (q_half.dtype == torch.bfloat16 and q_half.is_contiguous() and q_half.numel() == q_out.numel()),
          "head_norm_store: bad bfloat16 copy of the queries")
    for w in (wq, wk):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == dk and w.is_contiguous()), "head_norm_store: bad norm weight")
    width = (num_heads + num_kv_heads) * dk + (0 if v_off is None else num_kv_heads * dv)
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() >= width), "head_norm_store: bad bias")
    if store:
        _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype
              and tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dk)
              and tuple(v_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dv), "head_norm_store: bad pages")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "head_norm_store: bad block table")
    _check(lib().ms_head_norm_store(
        _ptr(proj), proj.stride(0), _ptr(bias), _ptr(wq), _ptr(wk), float(eps), float(temp_coef), int(temp_every), int(norm),
        _ptr(positions), _ptr(slot_of_token),
        _ptr(block_table), block_table.shape[1] if store else 0, k_pages.shape[0] if store else 0, k_pages.shape[2] if store else 0,
        _ptr(q_out), _ptr(q_half), _ptr(k_pages if store else None), _ptr(v_pages if store else None), _code(k_pages) if store else F32, t,
        num_heads, num_kv_heads, dk, dv, -1 if v_off is None else int(v_off), int(store), _stream()), "head_norm_store")
    return q_out


# ------------------------------------------------------------------------------------------- gated linear attention


def gla_decay(u, w2, b2, tau: float, out):
    """out[t, n] = exp(logsigmoid(w2[n, :] . u[t, :] + b2[n]) / tau): the decay sigmoid(z)^(1/tau), through its logarithm, in float32.
    u float32 [T, rank] (unit column stride); w2 [n, rank] float32 or bfloat16; b2 float32 [n] or None; out float32 [T, n]."""
    t, n = out.shape
    rank = w2.shape[1]
    _need(u.dtype == torch.float32 and u.stride(1) == 1 and u.shape[1] == rank and out.dtype == torch.float32 and out.is_contiguous()
          and w2.is_contiguous() and w2.shape[0] == n, "gla_decay: bad layout")
    _need(b2 is None or (b2.dtype == torch.float32 and b2.numel() == n), "gla_decay: bad bias")
    _check(lib().ms_gla_decay(_ptr(u), u.stride(0), _ptr(w2), _code(w2), _ptr(b2), rank, float(tau), _ptr(out), t, n, _stream()), "gla_decay")
    return out


def gla_scan(proj, q_off: int, k_off: int, v_off: int, decay, q_scale: float, state, cu_tokens, state_slots, slot_of_token, out,
             seqs: int, heads: int, dk: int, dv: int, narrow: bool = False):
    """The recurrence S <- diag(a_t) S + k_t v_t^T, o_t = S^T (q_t * q_scale), per sequence and head, over the rows of the
    step in order, from and to `state` (float32 [slots, heads, dk, dv]; a sequence's slot is state_slots[s]).
    proj float32 [T, ld] holds q, k (heads*dk each) and v (heads*dv) at the column offsets; decay (a) float32 [T, heads*dk];
    out float32 [T, heads*dv]; cu_tokens int32 [seqs + 1]; rows whose slot_of_token is negative are passed over.
    `narrow`: blocks of 8 value columns instead of 32 (more blocks a sequence: for steps with long portions); same bits."""
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and decay.dtype == torch.float32 and decay.is_contiguous()
          and out.dtype == torch.float32 and out.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous(),
          "gla_scan: bad layout")
    _need(tuple(state.shape[1:]) == (heads, dk, dv) and decay.shape[1] == heads * dk and out.shape[1] == heads * dv,
          "gla_scan: bad shapes")
    _need(cu_tokens.numel() >= seqs + 1 and state_slots.numel() >= seqs, "gla_scan: bad sequence lists")
    _check(lib().ms_gla_scan(_ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(decay), float(q_scale), _ptr(state),
                             _ptr(cu_tokens), _ptr(state_slots), _ptr(slot_of_token), _ptr(out), int(seqs), heads, dk, dv, int(narrow),
                             _stream()),
           "gla_scan")
    return out


def gla_output(o, gate, weight, eps: float, out, heads: int, dv: int):
    """out = o / rms(o) * weight (per head over dv, eps inside the root) * silu(gate).  o float32 [T, heads*dv] with unit
    column stride (any row stride); gate float32 [T, heads*dv] likewise, or None; weight float32 [dv] or None; out
    [T, heads*dv].  With one head and no gate: the RMS norm of the rows of a column range of a wider product."""
    t = o.shape[0]
    _need(o.dtype == torch.float32 and o.stride(1) == 1 and out.is_contiguous() and o.shape[1] == heads * dv
          and tuple(out.shape) == tuple(o.shape), "gla_output: bad layout")
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] == heads * dv), "gla_output: bad gate")
    _need(weight is None or (weight.dtype == torch.float32 and weight.numel() == dv), "gla_output: bad weight")
    _check(lib().ms_gla_output(_ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight), float(eps), _ptr(out),
                               _code(out), t, heads, dv, _stream()), "gla_output")
    return out


# ---------------------------------------------- a mixer of two halves: rotation with a cache of unequal widths, head gates, the gated delta rule


def norm_pair_mean(a, b, wa, wb, out, eps: float, scale: float = 0.5):
    """out = scale * (a / rms(a) * wa + b / rms(b) * wb), each root mean square over the row (eps inside the root), in float32.
    a, b, out float32 [T, d]; wa, wb float32 [d]."""
    t, d = out.shape
    _need(all(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (t, d) for x in (a, b, out)), "norm_pair_mean: bad rows")
    _need(all(w.dtype == torch.float32 and w.is_contiguous() and w.numel() == d for w in (wa, wb)), "norm_pair_mean: bad weights")
    _check(lib().ms_norm_pair_mean(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(out), t, d, float(eps), float(scale), _stream()), "norm_pair_mean")
    return out


def pair_weighted_sum(a, b, out, scale_a: float, scale_b: float, bias_a=None, bias_b=None):
    """out = scale_a * (a + bias_a) + scale_b * (b + bias_b) in float32.  a, b, out float32 [T, d]; the biases float32 [d] or None."""
    t, d = out.shape
    _need(all(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (t, d) for x in (a, b, out)), "pair_weighted_sum: bad rows")
    _need(all(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == d) for v in (bias_a, bias_b)),
          "pair_weighted_sum: bad biases")
    _check(lib().ms_pair_weighted_sum(_ptr(a), _ptr(b), _ptr(bias_a), _ptr(bias_b), _ptr(out), t, d, float(scale_a), float(scale_b), _stream()),
           "pair_weighted_sum")
    return out


# ------------------------------------------------------------------------------------------- the matrix memory (mLSTM cell)


def mm_state_floats(heads: int, dk: int, dv: int) -> int:
    """Floats of one request's state: per head the matrix with the normalizer as one more column, then the heads' stabilizers."""
    return heads * dk * (dv + 1) + heads


def mm_gates(proj, i_off: int, f_off: int, bias_i, bias_f, cap: float, state, cu_tokens, state_slots, slot_of_token, gates, seqs: int,
             heads: int, dk: int, dv: int):
    """The gates of a matrix memory over the rows of the step, sequence by sequence, in order: i = cap tanh(x_i / cap),
    f = logsigmoid(cap tanh(x_f / cap)), m_t = max(f_t + m_(t-1), i_t) from the m the slot holds (which is advanced),
    gates[t, h] = (exp(f_t + m_(t-1) - m_t), exp(i_t - m_t), m_t, 0).  proj float32 [T, ld] holds x_i at columns i_off + h and
    x_f at f_off + h; the biases float32 [heads] or None; state float32 [slots, mm_state_floats]; gates float32 [T, heads, 4]."""
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and gates.dtype == torch.float32 and gates.is_contiguous()
          and gates.numel() == proj.shape[0] * heads * 4, "mm_gates: bad layout")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] == mm_state_floats(heads, dk, dv),
          "mm_gates: bad state")
    _need(all(b is None or (b.dtype == torch.float32 and b.numel() == heads) for b in (bias_i, bias_f)), "mm_gates: bad biases")
    _need(cu_tokens.numel() >= seqs + 1 and state_slots.numel() >= seqs, "mm_gates: bad sequence lists")
    _check(lib().ms_mm_gates(_ptr(proj), proj.stride(0), int(i_off), int(f_off), _ptr(bias_i), _ptr(bias_f), float(cap), _ptr(state),
                             state.stride(0), heads * dk * (dv + 1), _ptr(cu_tokens), _ptr(state_slots), _ptr(slot_of_token), _ptr(gates),
                             int(seqs), heads, _stream()), "mm_gates")
    return gates


def mm_scan(proj, q_off: int, k_off: int, v_off: int, gates, q_scale: float, state, cu_tokens, state_slots, slot_of_token, out, seqs: int,
            heads: int, dk: int, dv: int, narrow: bool = False):
    """The recurrence S <- a_t S + b_t k_t v_t^T, n <- a_t n + b_t k_t per sequence and head over the rows of the step in
    order, from and to `state`; out[t, h, :dv] = S^T (q_t * q_scale), out[t, h, dv] = n . (q_t * q_scale).  proj float32 [T, ld]
    holds q, k (heads*dk each) and v (heads*dv) at the column offsets; gates float32 [T, heads, 4] as `mm_gates` leaves them;
    out float32 [T, heads, dv + 1].  `narrow`: blocks of 8 columns instead of 32 (for steps with long portions); same bits."""
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and gates.dtype == torch.float32 and gates.is_contiguous()
          and out.dtype == torch.float32 and out.is_contiguous() and out.numel() == proj.shape[0] * heads * (dv + 1), "mm_scan: bad layout")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] == mm_state_floats(heads, dk, dv),
          "mm_scan: bad state")
    _need(cu_tokens.numel() >= seqs + 1 and state_slots.numel() >= seqs, "mm_scan: bad sequence lists")
    _check(lib().ms_mm_scan(_ptr(proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(gates), float(q_scale), _ptr(state),
                            state.stride(0), _ptr(cu_tokens), _ptr(state_slots), _ptr(slot_of_token), _ptr(out), int(seqs), heads, dk, dv,
                            int(narrow), _stream()), "mm_scan")
    return out


def mm_output(o, gates, gate, weight, eps: float, out, heads: int, dv: int):
    """y = o[..., :dv] / (max(|o[..., dv]|, exp(-m)) + 1e-6), then out = y / rms(y) (per head over dv, eps inside the root)
    * weight * sigmoid(gate).  o float32 [T, heads, dv + 1] and gates float32 [T, heads, 4] as `mm_scan` and `mm_gates` leave
    them; gate float32 [T, heads*dv] with unit column stride (any row stride) or None; weight float32 [heads*dv] or None."""
    t = out.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.numel() == t * heads * (dv + 1) and out.is_contiguous()
          and tuple(out.shape) == (t, heads * dv) and gates.dtype == torch.float32 and gates.is_contiguous()
          and gates.numel() == t * heads * 4, "mm_output: bad layout")
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] == heads * dv), "mm_output: bad gate")
    _need(weight is None or (weight.dtype == torch.float32 and weight.numel() == heads * dv), "mm_output: bad weight")
    _check(lib().ms_mm_output(_ptr(o), _ptr(gates), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight), float(eps),
                              _ptr(out), _code(out), t, heads, dv, _stream()), "mm_output")
    return out


def softcap(x, cap: float):
    """x <- cap * tanh(x / cap) in place; x float32, contiguous."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "softcap: bad tensor")
    _check(lib().ms_softcap(_ptr(x), x.numel(), float(cap), _stream()), "softcap")
    return x


def head_gate_mul(x, gate, out, heads: int, dv: int):
    """out[r, h*dv + c] = x[r, h*dv + c] * sigmoid(gate[r, h]).  x, out [T, heads*dv] of one dtype (they may be the same tensor);
    gate float32 [T, heads] with unit column stride (any row stride)."""
    t = x.shape[0]
    _need(x.is_contiguous() and out.is_contiguous() and x.dtype == out.dtype and tuple(x.shape) == (t, heads * dv)
          and tuple(out.shape) == (t, heads * dv), "head_gate_mul: bad rows")
    _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and tuple(gate.shape) == (t, heads), "head_gate_mul: bad gate")
    _check(lib().ms_head_gate_mul(_ptr(x), _ptr(gate), gate.stride(0), _ptr(out), _code(x), t, heads, dv, _stream()), "head_gate_mul")
    return out


def rope_store(proj, cos_sin, rot: int, interleaved: bool, positions, slot_of_token, block_table, q_out, k_pages, v_pages, num_heads: int,
               num_kv_heads: int, dk: int, dv: int, store: bool = True, q_half=None, bias=None):
    """The first `rot` coordinates of every query and key head turned by the table's angles at the row's position (pairs
    (i, i + rot/2), or (2i, 2i + 1) when `interleaved`); q to q_out (float32 [T, Hq*dk]) and, optionally, to a bfloat16 copy;
    the turned keys into k_pages [pages, Hkv, page, dk] and the values into v_pages [pages, Hkv, page, dv].  proj float32
    [T, >= Hq*dk + Hkv*(dk + dv)] = [q | k | v]; cos_sin float32 [positions, rot/2, 2] (None when rot is 0); `bias` (float32,
    one entry per column of q | k | v, or None) is added to the product as it is read."""
    t = q_out.shape[0]
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous()
                           and bias.numel() == num_heads * dk + num_kv_heads * (dk + dv)), "rope_store: bad bias")
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.dtype == torch.float32 and q_out.is_contiguous()
          and q_out.numel() == t * num_heads * dk, "rope_store: bad layout")
    _need(q_half is None or (q_half.dtype == torch.bfloat16 and q_half.is_contiguous() and q_half.numel() == q_out.numel()),
          "rope_store: bad bfloat16 copy of the queries")
    _need(rot == 0 or (cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
                       and tuple(cos_sin.shape[1:]) == (rot // 2, 2)), "rope_store: bad table of angles")
    if store:
        _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype
              and tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dk)
              and tuple(v_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], dv), "rope_store: bad pages")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "rope_store: bad block table")
    _check(lib().ms_rope_store(
        _ptr(proj), proj.stride(0), _ptr(bias), _ptr(cos_sin if rot else None), int(rot), int(bool(interleaved)), cos_sin.shape[0] if rot else 0,
        _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1] if store else 0, k_pages.shape[0] if store else 0,
        k_pages.shape[2] if store else 0, _ptr(q_out), _ptr(q_half), _ptr(k_pages if store else None), _ptr(v_pages if store else None),
        _code(k_pages) if store else F32, t, num_heads, num_kv_heads, dk, dv, int(store), _stream()), "rope_store")
    return q_out


def gdr_prepare(proj, x_off: int, b_off: int, a_off: int, conv_w, a_log, dt_bias, state, conv_off: int, cu_tokens, seq_of_token,
                slot_of_token, qkv, bg, heads: int, groups: int, dk: int, dv: int, q_scale: float):
    """What the gated delta rule's recurrence reads, from the step's input product: the short causal convolution (weights
    conv_w float32 [C, taps], last column the current token's; the inputs before the step's first row come from the
    request's state) and SiLU of the C = 2*groups*dk + heads*dv channels [q | k | v] at column x_off of proj; q and k heads
    as unit vectors (x / sqrt(sum x^2 + 1e-6)), q times q_scale; beta = sigmoid(proj[:, b_off + h]); g = exp(-exp(a_log[h]) *
    softplus(proj[:, a_off + h] + dt_bias[h])).  qkv float32 [T, C] and bg float32 [T, 2*heads] (beta | g) are written.
    state float32 [slots, stride]: a slot's last taps - 1 inputs lie from conv_off on, [taps - 1, C], oldest first."""
    t, c = qkv.shape
    taps = conv_w.shape[1]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and qkv.dtype == torch.float32 and qkv.is_contiguous()
          and bg.dtype == torch.float32 and bg.is_contiguous() and tuple(bg.shape) == (t, 2 * heads)
          and c == 2 * groups * dk + heads * dv, "gdr_prepare: bad layout")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == c, "gdr_prepare: bad convolution weights")
    _need(all(v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads for v in (a_log, dt_bias)), "gdr_prepare: bad head constants")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
          and state.shape[1] >= conv_off + (taps - 1) * c, "gdr_prepare: bad state")
    _check(lib().ms_gdr_prepare(_ptr(proj), proj.stride(0), int(x_off), int(b_off), int(a_off), _ptr(conv_w), taps, _ptr(a_log), _ptr(dt_bias),
                                _ptr(state), state.shape[1], int(conv_off), _ptr(cu_tokens), _ptr(seq_of_token), _ptr(slot_of_token),
                                _ptr(qkv), _ptr(bg), t, heads, groups, dk, dv, float(q_scale), _stream()), "gdr_prepare")
    return qkv, bg


def gdr_conv_update(proj, x_off: int, taps: int, channels: int, state, conv_off: int, cu_tokens, state_slots, slot_of_token, seqs: int):
    """After `gdr_prepare`: every sequence's last taps - 1 inputs (of its state's, then the step's) become its state's."""
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
          and state.dim() == 2 and state.shape[1] >= conv_off + (taps - 1) * channels, "gdr_conv_update: bad layout")
    _check(lib().ms_gdr_conv_update(_ptr(proj), proj.stride(0), int(x_off), int(taps), _ptr(state), state.shape[1], int(conv_off),
                                    _ptr(cu_tokens), _ptr(state_slots), _ptr(slot_of_token), int(seqs), int(channels), _stream()),
           "gdr_conv_update")


def gdr_scan(qkv, bg, state, cu_tokens, state_slots, slot_of_token, out, seqs: int, heads: int, groups: int, dk: int, dv: int,
             narrow: bool = False):
    """The recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per sequence and value head (q/k head
    h // (heads / groups)), over the rows of the step in order, from and to `state` (float32 [slots, stride], the matrices
    [heads, dk, dv] at the start of a slot's row).  qkv, bg as `gdr_prepare` leaves them; out float32 [T, heads*dv].
    `narrow`: blocks of 8 value columns instead of 32 (more blocks a sequence); same bits."""
    t = qkv.shape[0]
    _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[1] == 2 * groups * dk + heads * dv and bg.dtype == torch.float32
          and bg.is_contiguous() and tuple(bg.shape) == (t, 2 * heads) and out.dtype == torch.float32 and out.is_contiguous()
          and tuple(out.shape) == (t, heads * dv), "gdr_scan: bad layout")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] >= heads * dk * dv, "gdr_scan: bad state")
    _need(cu_tokens.numel() >= seqs + 1 and state_slots.numel() >= seqs, "gdr_scan: bad sequence lists")
    _check(lib().ms_gdr_scan(_ptr(qkv), _ptr(bg), _ptr(state), state.shape[1], _ptr(cu_tokens), _ptr(state_slots), _ptr(slot_of_token),
                             _ptr(out), int(seqs), heads, groups, dk, dv, int(narrow), _stream()), "gdr_scan")
    return out


# ------------------------------------------------------------------------------------------------ routed feed-forward


def moe_route(logits, top: int, ids, weights, bias=None):
    """Of each row's router logits (float32 [T, E], plus `bias` float32 [E] if given) the `top` largest (the lower index wins a tie), in descending order:
    ids int32 [T, top], weights float32 [T, top] = the softmax over the chosen logits only."""
    t, e = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and ids.dtype == torch.int32 and ids.is_contiguous()
          and weights.dtype == torch.float32 and weights.is_contiguous() and tuple(ids.shape) == (t, top) and tuple(weights.shape) == (t, top),
          "moe_route: bad arguments")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == e), "moe_route: bad bias")
    _check(lib().ms_moe_route(_ptr(logits), _ptr(bias), e, int(top), _ptr(ids), _ptr(weights), t, _stream()), "moe_route")
    return ids, weights


def moe_route_scored(logits, top: int, ids, weights, correction=None, groups: int = 1, keep: int = 1, scale: float = 1.0):
    """The choice by scores: s = sigmoid(logits) (float32 [T, E]); an expert is chosen by s + correction (float32 [E] or None),
    among the experts of the `keep` best of `groups` equal groups of neighbours (a group's score: the sum of its two largest
    choice scores; the lower index wins a tie); ids int32 [T, top] in descending order of the choice scores, weights float32
    [T, top] = the chosen experts' s over their sum (+ 1e-20), times `scale`."""
    t, e = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and ids.dtype == torch.int32 and ids.is_contiguous()
          and weights.dtype == torch.float32 and weights.is_contiguous() and tuple(ids.shape) == (t, top) and tuple(weights.shape) == (t, top),
          "moe_route_scored: bad arguments")
    _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == e),
          "moe_route_scored: bad correction")
    _check(lib().ms_moe_route_scored(_ptr(logits), _ptr(correction), e, int(top), int(groups), int(keep), float(scale), _ptr(ids),
                                     _ptr(weights), t, _stream()), "moe_route_scored")
    return ids, weights


def moe_gate_up_pairs(x, w_gate, w_up, ids, slot_of_token, h, activation: str):
    """h[t*top + j, :] = act(w_gate[e] x_t) * (w_up[e] x_t) with e = ids[t, j] (`w_up` None, experts without a gate:
    act(w_gate[e] x_t) alone).  x [T, d]; w_gate, w_up [E, ff, d];
    h [T*top, ff]; all of one dtype (float32 or bfloat16).  Rows with a negative slot get zeros."""
    t, d = x.shape
    experts, ff, _ = w_gate.shape
    top = ids.shape[1]
    _need(x.is_contiguous() and w_gate.is_contiguous() and h.is_contiguous() and ids.is_contiguous()
          and x.dtype == w_gate.dtype == h.dtype and w_gate.shape[2] == d
          and tuple(h.shape) == (t * top, ff) and ids.dtype == torch.int32 and ids.shape[0] == t, "moe_gate_up_pairs: bad arguments")
    _need(w_up is None or (w_up.is_contiguous() and w_up.dtype == x.dtype and tuple(w_up.shape) == (experts, ff, d)),
          "moe_gate_up_pairs: bad second matrix")
    step = max(1, 65535 // top)
    for t0 in range(0, t, step):
        n = min(step, t - t0)
        _check(lib().ms_moe_gate_up_pairs(_ptr(x[t0:]), _ptr(w_gate), _ptr(w_up), _ptr(ids[t0:]), _ptr(slot_of_token[t0:]), _ptr(h[t0 * top:]),
                                          _code(x), n, top, d, ff, experts, ACTIVATIONS[activation], _stream()), "moe_gate_up_pairs")
    return h


def moe_down_pairs(h, w_down, ids, weights, slot_of_token, y):
    """y[t, :] = sum_j weights[t, j] * (w_down[ids[t, j]] h[t*top + j, :]), j ascending, in float32.  h [T*top, ff];
    w_down [E, d, ff] of h's dtype; y float32 [T, d]."""
    t, d = y.shape
    experts, _, ff = w_down.shape
    top = ids.shape[1]
    _need(h.is_contiguous() and w_down.is_contiguous() and y.is_contiguous() and y.dtype == torch.float32 and h.dtype == w_down.dtype
          and tuple(h.shape) == (t * top, ff) and w_down.shape[1] == d and weights.dtype == torch.float32 and weights.is_contiguous()
          and tuple(weights.shape) == (t, top) and ids.dtype == torch.int32 and ids.is_contiguous(), "moe_down_pairs: bad arguments")
    for t0 in range(0, t, 65535):
        n = min(65535, t - t0)
        _check(lib().ms_moe_down_pairs(_ptr(h[t0 * top:]), _ptr(w_down), _ptr(ids[t0:]), _ptr(weights[t0:]), _ptr(slot_of_token[t0:]),
                                       _ptr(y[t0:]), _code(h), n, top, d, ff, experts, _stream()), "moe_down_pairs")
    return y


def moe_grouped_supports(d: int, ff: int, experts: int) -> bool:
    """Whether the sorted, tiled form of the routed feed-forward covers the sizes (both widths multiples of 32)."""
    return bool(lib().ms_moe_grouped_supports(int(d), int(ff), int(experts)))


def moe_grouped_scratch_ints(pairs: int, experts: int) -> int:
    fn = lib().ms_moe_grouped_scratch_ints
    fn.restype = c_longlong
    fn.argtypes = [c_int, c_int]
    return int(fn(int(pairs), int(experts)))


def moe_grouped(x, w_gate, w_up, w_down, ids, weights, slot_of_token, scratch, h, z, y, activation: str):
    """The routed feed-forward for many rows, bfloat16, on the tensor cores: the (token, expert) pairs sorted by expert on
    the device, every expert's rows through its matrices in tiles, the pairs' results summed per token with the router's
    weights (j ascending).  x [T, d]; w_gate, w_up [E, ff, d]; w_down [E, d, ff]; ids int32, weights float32 [T, top];
    scratch int32 (`moe_grouped_scratch_ints`), h bfloat16 [T*top, ff], z float32 [T*top, d]; y float32 [T, d]."""
    t, d = x.shape
    experts, ff, _ = w_gate.shape
    top = ids.shape[1]
    bf = torch.bfloat16
    _need(x.dtype == bf and w_gate.dtype == bf and w_down.dtype == bf and h.dtype == bf and x.is_contiguous()
          and w_gate.is_contiguous() and w_down.is_contiguous() and h.is_contiguous(), "moe_grouped: bad operands")
    _need(w_up is None or (w_up.dtype == bf and w_up.is_contiguous() and tuple(w_up.shape) == (experts, ff, d)),
          "moe_grouped: bad second matrix")  # (None: experts without a gate, h = act(w_gate x))
    _need(tuple(w_down.shape) == (experts, d, ff) and w_gate.shape[2] == d
          and tuple(h.shape) == (t * top, ff) and tuple(z.shape) == (t * top, d) and tuple(y.shape) == (t, d)
          and z.dtype == torch.float32 and y.dtype == torch.float32 and z.is_contiguous() and y.is_contiguous(), "moe_grouped: bad shapes")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
          and tuple(weights.shape) == (t, top) and scratch.dtype == torch.int32
          and scratch.numel() >= moe_grouped_scratch_ints(t * top, experts), "moe_grouped: bad lists")
    _check(lib().ms_moe_grouped(_ptr(x), _ptr(w_gate), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(slot_of_token), _ptr(scratch),
                                _ptr(h), _ptr(z), _ptr(y), t, top, d, ff, experts, ACTIVATIONS[activation], _stream()), "moe_grouped")
    global _launches
    _launches += 3  # the sort, two products and the sum are four launches
    return y


def apply_logit_offsets(logits, row_ptr, tokens, amounts):
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "apply_logit_offsets: bad logits")
    _need(row_ptr.dtype == torch.int32 and tokens.dtype == torch.int32 and amounts.dtype == torch.float32,
          "apply_logit_offsets: bad dtypes")
    _check(
        lib().ms_apply_logit_offsets(_ptr(logits), rows, vocab, _ptr(row_ptr), _ptr(tokens), _ptr(amounts), _stream()),
        "apply_logit_offsets",
    )
    return logits


def sample(logits, temperature, top_k, top_p, rng_state, out_token, out_logprob):
    """One token per row.  rng_state int64 [R] holds the SplitMix64 states and is advanced in place."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and top_k.dtype == torch.int32, "sample: bad dtypes")
    _need(rng_state.dtype == torch.int64 and out_token.dtype == torch.int32 and out_logprob.dtype == torch.float32,
          "sample: bad dtypes")
    _need(min(temperature.numel(), top_k.numel(), top_p.numel(), rng_state.numel(), out_token.numel(),
              out_logprob.numel()) >= rows, "sample: per-row arrays are shorter than the rows")
    _check(
        lib().ms_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(rng_state),
                        _ptr(out_token), _ptr(out_logprob), _stream()),
        "sample",
    )
    return out_token


TOP_LOGPROBS_MAX = 20


def top_logprobs(logits, temperature, want, out_token, out_logprob):
    """The want[r] (at most 20) most probable tokens of every row and their log-probabilities at the row's
    temperature, ranked; out_token int32 and out_logprob float32 are [rows, 20]."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "top_logprobs: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and want.dtype == torch.int32 and min(temperature.numel(), want.numel()) >= rows,
          "top_logprobs: bad per-row arrays")
    _need(out_token.dtype == torch.int32 and out_logprob.dtype == torch.float32 and out_token.is_contiguous() and
          out_logprob.is_contiguous() and min(out_token.numel(), out_logprob.numel()) >= rows * TOP_LOGPROBS_MAX,
          "top_logprobs: the outputs must be [rows, 20]")
    _check(lib().ms_top_logprobs(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(want), _ptr(out_token), _ptr(out_logprob),
                                 _stream()), "top_logprobs")
