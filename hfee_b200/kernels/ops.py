"""Python face of the sm_100a kernel library: one function per kernel, taking torch
tensors (used only as typed device buffers) and launching on torch's current CUDA
stream.  There is no other implementation behind these functions: without a
CUDA device of compute capability 10.x and the built library they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing, cannot be loaded or refused a call."""


_LIB: Optional[ctypes.CDLL] = None
_DT = {torch.float32: 0, torch.bfloat16: 1}

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_SIGNATURES = {
    "hfee_embed": [_P, _I, _P, _P, _P, _P, _I, _I, _I, _F, _P],
    "hfee_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "hfee_rope_table": [_P, _P, _P, _I, _I, _P],
    "hfee_rope_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "hfee_swiglu": [_P, _I, _P, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_stream": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_stream_norm": [_P, _L, _P, _P, _F, _I, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_tcgen05": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _L, _P, _P],
    "hfee_gemm_tcgen05_stream_k": [_I, _I, _I, _I, _L],
    "hfee_gemm_tcgen05_pair": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_tcgen05_rope": [_P, _L, _P, _L, _I, _I, _I, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_tcgen05_rope_supports": [_I, _I],
    "hfee_gemm_skinny": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _L, _P, _P],
    "hfee_gemm_skinny_splits": [_I, _I, _I, _L],
    "hfee_gemm_ring": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_ring_supports": [_I, _I, _I, _I],
    "hfee_attention_tc": [_P, _I, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "hfee_attention_tc_supports": [_I, _I, _I, _I],
    "hfee_attention_mma": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "hfee_attention_mma_rope": [_P, _I, _P, _I, _I, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "hfee_gemm_simt": [_P, _L, _P, _L, _I, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_attention_simt": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "hfee_attention_simt_masked": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _L, _I, _P],
    "hfee_attention_sigmoid_mma": [_P, _L, _P, _P, _P, _I, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _L, _P],
    "hfee_attention_sigmoid_mma_supports": [_I, _I, _I],
    "hfee_short_conv": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P],
    "hfee_short_conv_launches": [_I, _I, _I],
    "hfee_linear_attention": [_P, _P, _P, _L, _I, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P],
    "hfee_linear_attention_chunked": [_P, _P, _P, _L, _I, _P, _P, _P, _P, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "hfee_rmsnorm_add": [_P, _L, _P, _P, _I, _I, _F, _I, _P, _L, _I, _P],
    "hfee_rmsnorm_add_norm": [_P, _L, _P, _P, _I, _I, _F, _I, _P, _F, _I, _P, _L, _I, _P],
    "hfee_norm_gate": [_P, _L, _P, _F, _P, _L, _P, _L, _I, _I, _I, _P],
    "hfee_gated_act": [_P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_scale_f32": [_P, _L, _I, _I, _F, _P],
    "hfee_cast_rows": [_P, _P, _L, _I, _I, _I, _P],
    "hfee_qk_norm_rope_cache": [_P, _L, _P, _P, _F, _P, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "hfee_attention_simt_general": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _L, _I, _I, _P],
    "hfee_rope_norm_cache": [_P, _L, _I, _I, _P, _I, _F, _P, _P, _I, _I, _I, _I, _I, _P, _L, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I,
                             _I, _I, _I, _P, _I, _P, _I, _I, _P],
    "hfee_latent_norm_rope_cache": [_P, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _P, _P, _L, _P, _P, _I, _I, _P],
    "hfee_latent_attention_mma": [_P, _L, _P, _P, _I, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _I, _P],
    "hfee_latent_attention_mma_supports": [_I, _I, _I],
    "hfee_head_linear": [_P, _L, _I, _I, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P, _L, _I, _P],
    "hfee_conv_act": [_P, _L, _I, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P],
    "hfee_attention_simt_distance": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _L, _I,
                                     _P, _P, _F, _I, _P],
    "hfee_attention_mma_distance": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _F, _I, _I,
                                    _P, _P],
    "hfee_attention_mma_distance_tile": [_I, _I],
    "hfee_add_sinusoid": [_P, _P, _I, _I, _F, _P],
    "hfee_softcap": [_P, _L, _I, _I, _F, _P],
    "hfee_clamped_glu": [_P, _L, _P, _L, _I, _I, _I, _F, _F, _F, _I, _P],
    "hfee_scaled_add_norm": [_P, _F, _P, _P, _F, _P, _L, _I, _I, _I, _P],
    "hfee_depth_average": [_P, _P, _F, _P, _L, _P, _I, _I, _I, _P],
    "hfee_mingru": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_selective_scan": [_P, _L, _P, _L, _P, _L, _I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _F, _I, _I, _P],
    "hfee_moe_route": [_P, _I, _I, _I, _F, _P, _P, _P],
    "hfee_moe_plan": [_P, _I, _I, _P, _P, _P, _P, _I, _P],
    "hfee_moe_gate_up": [_P, _L, _I, _P, _P, _L, _I, _I, _P, _P, _P, _P, _P, _L, _F, _F, _F, _I, _I, _P],
    "hfee_moe_down": [_P, _L, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P],
    "hfee_moe_combine": [_P, _P, _P, _I, _I, _P, _I, _I, _P],
    "hfee_moe_plan_tiles": [_P, _I, _I, _I, _P, _P, _P, _I, _P],
    "hfee_moe_gather_rows": [_P, _L, _I, _P, _P, _I, _P, _L, _I, _I, _P],
    "hfee_gemm_tcgen05_grouped": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _I, _F, _F, _F, _P, _P],
    "hfee_gemm_tcgen05_pair_clamped": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _F, _F, _F, _P, _P],
    "hfee_embed_bigram": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _P],
    "hfee_remember_tokens": [_P, _P, _P, _P, _P, _I, _P, _P],
    "hfee_layernorm": [_P, _P, _P, _P, _P, _L, _I, _I, _I, _F, _P],
    "hfee_add_bias": [_P, _L, _P, _I, _I, _P],
    "hfee_attention_prepare": [_P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _F, _P, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I,
                               _I, _I, _I, _I, _P],
    "hfee_attention_simt_sink": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _L, _I,
                                 _P, _P, _F, _P, _I, _P],
    "hfee_attention_mma_general": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P, _F, _I,
                                   _I, _P, _P],
    "hfee_gated_recurrence": [_I, _P, _P, _P, _L, _I, _P, _L, _P, _F, _F, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_gated_recurrence_chunked": [_I, _P, _P, _P, _L, _I, _P, _L, _P, _F, _F, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P, _L, _P],
    "hfee_head_norm_gate_scaled": [_P, _L, _P, _I, _F, _P, _L, _P, _L, _I, _I, _I, _I, _F, _I, _P],
    "hfee_moe_combine_extra": [_P, _P, _P, _I, _I, _P, _I, _I, _P, _P, _L, _P],
    "hfee_moe_route_grouped": [_P, _L, _I, _I, _I, _I, _I, _F, _P, _P, _P],
    "hfee_conv_act_launches": [_I, _I, _I],
    "hfee_delta_rule": [_P, _L, _I, _I, _I, _P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _P, _L, _P],
    "hfee_head_norm_gate": [_P, _L, _P, _F, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_unary_act": [_P, _L, _P, _L, _I, _I, _I, _I, _P],
    "hfee_head_gate": [_P, _L, _P, _L, _I, _I, _I, _I, _P],
    "hfee_sample": [_P, _L, _I, _I, _P, _P, _P, _L, _P, _P, _P, _P],
    "hfee_argmax": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P],
    "hfee_sample_chain": [_P, _L, _I, _I, _P, _P, _P, _I, _P, _I, _P, _L, _P, _P, _P],
}


def library() -> ctypes.CDLL:
    """Load (building first if needed) the kernel library; raises if impossible."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: hfee_b200 runs on sm_100a GPUs only and has no CPU path")
    try:
        path = _build.build()
        lib = ctypes.CDLL(path)
    except (OSError, _build.KernelBuildError) as e:
        raise KernelLibraryError(f"cannot load the sm_100a kernel library: {e}") from e
    lib.hfee_last_error.restype = ctypes.c_char_p
    lib.hfee_device_is_sm100.restype = _I
    lib.hfee_sm_count.restype = _I
    lib.hfee_set_carveout.restype = _I
    lib.hfee_set_carveout.argtypes = [_I]
    lib.hfee_gemm_skinny_splits.restype = _I
    lib.hfee_attention_tc_supports.restype = _I
    lib.hfee_linear_attention_chunked_workspace.restype = _L
    lib.hfee_linear_attention_chunked_workspace.argtypes = [_I, _I, _I, _I, _I]
    lib.hfee_delta_rule_workspace.restype = _L
    lib.hfee_delta_rule_workspace.argtypes = [_I, _I, _I, _I, _I]
    lib.hfee_gated_recurrence_workspace.restype = _L
    lib.hfee_gated_recurrence_workspace.argtypes = [_I, _I, _I, _I, _I]
    lib.hfee_moe_tile_rows.restype = _I
    lib.hfee_moe_tile_rows.argtypes = []
    for name, sig in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"{path} lacks the symbol {name}") from e
        fn.argtypes = sig
        fn.restype = _I
    if not lib.hfee_device_is_sm100():
        major, minor = torch.cuda.get_device_capability()
        raise KernelLibraryError(f"the kernels are built for sm_100a only; this device is sm_{major}{minor}")
    _LIB = lib
    return lib


def set_carveout(percent: Optional[int]) -> Optional[int]:
    """The split between shared memory and L1 that the launches that follow ask for: percent of the
    SM's shared-memory maximum, or None for the driver's choice per kernel.  Returns the setting before.
    A chain of short kernels runs fastest when all of them ask for the same split."""
    before = library().hfee_set_carveout(-1 if percent is None else int(percent))
    return None if before < 0 else before


def sm_count() -> int:
    """Streaming multiprocessors of the current device, as the kernels' launchers see them."""
    global _SMS
    if _SMS is None:
        n = library().hfee_sm_count()
        if n <= 0:
            raise KernelLibraryError("cannot ask the device for its number of SMs")
        _SMS = n
    return _SMS


_SMS: Optional[int] = None


def loaded_library_path() -> Optional[str]:
    return _LIB._name if _LIB is not None else None


_LAUNCHES = 0

# Measuring what a class of kernels costs inside a step: the parts name the class of their next
# launches with tag(); leave_out(classes) makes every launch of those classes a no-op (the results
# are then wrong, the timing of the rest is not), and the difference of the step time with and
# without a class is what it costs in place, overlap with its neighbours included.
_TAG = ""
_LEFT_OUT: frozenset = frozenset()


def tag(name: str) -> str:
    """Name the class of the launches that follow; returns the class named before."""
    global _TAG
    before, _TAG = _TAG, name
    return before


def leave_out(classes=()) -> None:
    global _LEFT_OUT
    _LEFT_OUT = frozenset(classes)


def _measurable(fn):
    import functools

    @functools.wraps(fn)
    def call(*args, **kwargs):
        if _LEFT_OUT and _TAG in _LEFT_OUT:
            # a product left out still lets the norm in front of it run, unless the kernel would have
            # computed that norm itself
            if args and not isinstance(args[0], torch.Tensor) and hasattr(args[0], "tensor") and not _norm_fusable(args[0], args[1]):
                args[0].tensor()
            return None
        return fn(*args, **kwargs)
    return call


def launch_count() -> int:
    """Kernels launched through this module so far (a graph replay counts its kernels)."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, lib: ctypes.CDLL) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if code != 0:
        raise KernelLibraryError(lib.hfee_last_error().decode() or f"kernel call failed with code {code}")


_STREAM_HELD: Optional[int] = None


def _stream() -> int:
    return _STREAM_HELD if _STREAM_HELD is not None else torch.cuda.current_stream().cuda_stream


class stream_held:
    """``with ops.stream_held():`` every launch inside goes to the stream that is current at entry,
    asked of torch once instead of once per launch (a third of the host's time for a prompt pass of a
    16-layer model went into that question).  Nothing inside may change the current stream."""

    def __enter__(self):
        global _STREAM_HELD
        self.before = _STREAM_HELD
        _STREAM_HELD = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _STREAM_HELD
        _STREAM_HELD = self.before
        return False


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelLibraryError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16") from None


def _rows(t: torch.Tensor, what: str) -> int:
    """Leading dimension (in elements) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelLibraryError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                                 f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous() or not t.is_cuda):
        raise KernelLibraryError(f"{what}: expected a contiguous int32 CUDA tensor")


# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, slot_of_token: Optional[torch.Tensor] = None,
          feedback: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[i,:] = table[tokens[i],:] * scale widened to float32.  With ``feedback`` (int32 per request slot)
    a negative token id stands for ``feedback[slot_of_token[i]]``: the token last sampled on the
    device for that request."""
    lib = library()
    _i32(tokens, "embed tokens"); _i32(slot_of_token, "slot_of_token"); _i32(feedback, "feedback")
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert feedback is None or slot_of_token is not None
    n, width = out.shape
    _check(lib.hfee_embed(table.data_ptr(), _dt(table), tokens.data_ptr(), _ptr(slot_of_token), _ptr(feedback),
                          out.data_ptr(), n, width, table.shape[0], float(scale), _stream()), lib)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, add_unit: bool = False) -> None:
    """out[r,:] = x[rows[r] or r,:] * rsqrt(mean(x^2)+eps) * weight (float32 math)."""
    lib = library()
    _i32(rows, "rmsnorm rows")
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == x.shape[1]
    n, width = out.shape
    _check(lib.hfee_rmsnorm(x.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(), _dt(out), n, width,
                            float(eps), int(add_unit), _stream()), lib)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[i, j] = (cos, sin)(positions[i] * inv_freq[j]), computed in float64."""
    lib = library()
    _i32(positions, "rope positions")
    assert inv_freq.dtype == torch.float64 and out.dtype == torch.float32 and out.is_contiguous()
    n, half = positions.numel(), inv_freq.numel()
    assert out.numel() == n * half * 2
    _check(lib.hfee_rope_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), n, half, _stream()), lib)


def rope_cache_write(qkv: torch.Tensor, cs: Optional[torch.Tensor], positions: torch.Tensor,
                     slot_of_token: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                     v_pool: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int,
                     heads: int, kv_heads: int, head_dim: int, rope_dim: int, interleaved: bool) -> None:
    """Rotate q into ``q_out`` and k into its cache page, copy v to its page.
    ``qkv`` rows are [q heads | k heads | v heads]; pools are [pages, kv_heads, page_size, head_dim]."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = qkv.shape[0]
    want = (heads + 2 * kv_heads) * head_dim if k_pool is not None else heads * head_dim
    assert qkv.shape[1] == want and q_out.dtype == qkv.dtype
    if k_pool is not None:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
        assert k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), (k_pool.shape, kv_heads, page_size, head_dim)
    _check(lib.hfee_rope_cache_write(qkv.data_ptr(), _rows(qkv, "qkv"), _ptr(cs), positions.data_ptr(),
                                     slot_of_token.data_ptr(), q_out.data_ptr(), _rows(q_out, "q_out"),
                                     _ptr(k_pool), _ptr(v_pool), block_table.data_ptr(), block_table.shape[1],
                                     page_size, n, heads, kv_heads, head_dim, rope_dim, int(interleaved),
                                     _dt(qkv), _stream()), lib)


# Prompt portions: rotation and cache write in the epilogue of the q/k/v product instead of a pass of
# their own over the projection (prompt of 2,048 tokens, benchmark model: 11 us per layer less).
FUSE_ROPE_INTO_QKV = True
QKV_ROPE_MIN_TOKENS = 65         # from here on linear() takes the large-tile tcgen05 kernel anyway


def qkv_rope_fusable(a_dtype: torch.dtype, n: int, w: torch.Tensor, head_dim: int, rope_dim: int,
                     cs: Optional[torch.Tensor], q_out: torch.Tensor) -> bool:
    """True when :func:`linear_rope_cache` takes this step."""
    return (FUSE_ROPE_INTO_QKV and USE_TCGEN05 and a_dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and n >= QKV_ROPE_MIN_TOKENS and head_dim in (64, 128) and (cs is None or rope_dim == head_dim)
            and w.shape[1] % 8 == 0 and _rows(w, "w") % 8 == 0 and w.data_ptr() % 16 == 0
            and _rows(q_out, "q_out") % 8 == 0 and q_out.data_ptr() % 16 == 0)


def linear_rope_cache(a: torch.Tensor, w: torch.Tensor, cs: Optional[torch.Tensor], positions: torch.Tensor,
                      slot_of_token: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                      v_pool: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int, heads: int,
                      kv_heads: int, head_dim: int, interleaved: bool) -> None:
    """``a @ w.T`` with rows of ``w`` = [q heads | k heads | v heads] ([q heads] when the pools are
    None), rotated by ``cs`` ([n, head_dim/2, 2] cosines and sines) in the product's epilogue: queries
    to ``q_out``, keys and values to the cache pages of (slot, position).  Nothing else is stored."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n, k = a.shape
    want = (heads + 2 * kv_heads) * head_dim if k_pool is not None else heads * head_dim
    assert w.shape == (want, k) and a.dtype == w.dtype == q_out.dtype == torch.bfloat16
    assert a.data_ptr() % 16 == 0 and _rows(a, "a") % 8 == 0 and q_out.shape[0] == n
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * head_dim)
    if k_pool is not None:
        assert k_pool.dtype == v_pool.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_gemm_tcgen05_rope(a.data_ptr(), _rows(a, "a"), w.data_ptr(), _rows(w, "w"), n, want, k, _ptr(cs),
                                      positions.data_ptr(), slot_of_token.data_ptr(), q_out.data_ptr(),
                                      _rows(q_out, "q_out"), _ptr(k_pool), _ptr(v_pool), block_table.data_ptr(),
                                      block_table.shape[1], page_size, heads, kv_heads, head_dim, int(interleaved),
                                      _status().data_ptr(), _stream()), lib)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, granule: Optional[int] = None) -> None:
    """out[i, c] = silu(gate) * up.  Columns of ``gate_up`` come in groups of ``granule`` gate
    columns followed by ``granule`` up columns (default: all gate columns, then all up columns)."""
    lib = library()
    n, inter = out.shape
    assert gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype
    _check(lib.hfee_swiglu(gate_up.data_ptr(), _rows(gate_up, "gate_up"), out.data_ptr(), _rows(out, "swiglu out"),
                           n, inter, int(granule or inter), _dt(out), _stream()), lib)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T on the CUDA cores with float32 accumulation, k in order."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n) and a.dtype == w.dtype
    _check(lib.hfee_gemm_simt(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), _dt(a),
                              out.data_ptr(), _rows(out, "gemm out"), _dt(out), int(accumulate), m, n, k,
                              _stream()), lib)


STREAM_MAX_TOKENS = 64
USE_TCGEN05 = True
EPI_STORE, EPI_ACCUM, EPI_SWIGLU, EPI_GEGLU, EPI_RELU2 = 0, 1, 2, 4, 5      # 5 (tcgen05 kernels only): store relu(x)^2
EPI_GATED = (EPI_SWIGLU, EPI_GEGLU)         # out = act(gate) * up over rows of w interleaved as [4 gate | 4 up]


def _streamable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= STREAM_MAX_TOKENS and a.shape[1] % 8 == 0
            and _rows(a, "a") % 8 == 0 and _rows(w, "w") % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 64 rows of ``a`` (bfloat16), streaming ``w`` once through
    mma.sync tiles.  ``epilogue``: store, accumulate into float32 ``out``, or SwiGLU over rows
    of ``w`` interleaved as [4 gate | 4 up] (then ``out`` is [m, n/2])."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    _check(lib.hfee_gemm_stream(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _stream()), lib)


_STATUS: Optional[torch.Tensor] = None


def gemm_ring(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 8 rows of ``a`` (bfloat16, width a multiple of 64): one CTA per SM
    streams its share of the rows of ``w`` through a ring of TMA boxes.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    _check(lib.hfee_gemm_ring(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                              _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _status().data_ptr(), _stream()), lib)


_RING_TAKES: dict = {}


def ring_takes(m: int, n: int, k: int, epilogue: int) -> bool:
    key = (m, n, k, epilogue)
    if key not in _RING_TAKES:
        _RING_TAKES[key] = bool(library().hfee_gemm_ring_supports(*key))
    return _RING_TAKES[key]


def _status() -> torch.Tensor:
    global _STATUS
    if _STATUS is None:
        _STATUS = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _STATUS


def check_status() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
    if _STATUS is not None and int(_STATUS.item()) != 0:
        _STATUS.zero_()
        raise KernelLibraryError("a tcgen05 kernel gave up waiting on a barrier; its output is invalid")


def _tensor_core_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and _rows(a, "a") % 8 == 0
            and _rows(w, "w") % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE,
                 block_n: Optional[int] = None, stream_k: Optional[bool] = None) -> None:
    """out (+)= a @ w.T with tcgen05.mma tiles of 128 x block_n fed by TMA (bfloat16 in, float32
    accumulation in tensor memory).  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    tiles_256 = 0
    if block_n is None:
        # wide tiles need a third less shared-memory feed per flop (a 128-wide tile's feed rate is at
        # the L2 -> shared-memory limit); narrow ones fill the SMs when there are few tiles.  Measured
        # at M = N = 2048 (128 wide tiles on 148 SMs): K = 8192 takes 61 us wide, 95 us narrow.
        tiles_256 = -(-m // 128) * -(-n // 256)
        block_n = 256 if tiles_256 >= 96 else 128
        # 192 wide where that saves a round of tiles: 16 x 12 tiles of 256 are two rounds on 148 SMs
        # with the second a third full, 16 x 16 tiles of 192 are two rounds of three quarters the work
        if block_n == 256 and n % 192 == 0:
            rounds = lambda bn: -(-(-(-m // 128) * -(-n // bn)) // sm_count())
            if rounds(192) * 192 * 1.05 < rounds(256) * 256:
                block_n = 192
    if USE_PAIRS and block_n == 256 and m > 128 and tiles_256 >= 96 and (epilogue != EPI_STORE or n * k >= PAIR_STORE_MIN):
        gemm_tcgen05_pair(a, w, out, epilogue)
        return
    if stream_k is None:
        stream_k = USE_STREAM_K
    ws, flags = _stream_k_workspace() if stream_k else (None, None)
    _check(lib.hfee_gemm_tcgen05(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                 _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, block_n,
                                 _status().data_ptr(), _ptr(ws), ws.numel() if ws is not None else 0, _ptr(flags),
                                 _stream()), lib)


# Two CTAs on a tile of 256 x 256 (cta_group::2) where the single-CTA kernel would take tiles of
# 128 x 256: measured at 2,048 tokens, gate/up of the benchmark model 102 -> 90 us (1,527 TFLOP/s), down
# projection 57 -> 50 us, output projection 16.6 -> 17.0 us.
USE_PAIRS = True
PAIR_STORE_MIN = 1 << 62        # plain stores: the single-CTA kernel until measured otherwise


def gemm_tcgen05_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """:func:`gemm_tcgen05` with two CTAs on each tile of 256 x 256 (``cta_group::2``): each CTA loads
    its own 128 rows of ``a`` and half of the tile's rows of ``w``.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    _check(lib.hfee_gemm_tcgen05_pair(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                      _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _status().data_ptr(),
                                      _stream()), lib)


USE_STREAM_K = True
_STREAM_K_WS = None


def _stream_k_workspace():
    """One float32 tile of 128 x 256 per SM for the partial tiles of products split by K blocks, and
    two flag words per SM (zero at the start; every launch leaves them zero).  Made once, 19 MiB."""
    global _STREAM_K_WS
    if _STREAM_K_WS is None:
        _STREAM_K_WS = (torch.empty(sm_count() * 128 * 256, dtype=torch.float32, device="cuda"),
                        torch.zeros(2 * sm_count(), dtype=torch.int32, device="cuda"))
    return _STREAM_K_WS


def gemm_stream_norm(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                     epilogue: int = EPI_STORE, rows: Optional[torch.Tensor] = None, add_unit: bool = False) -> None:
    """:func:`gemm_stream` with the RMS norm fused in front: the token operand is
    bf16(x[rows] * rsqrt(mean(x^2) + eps) * norm_weight) made on the fly from float32 rows.  At most
    8 rows and a width of at most 2,048 (the kernel that keeps the tokens in registers)."""
    lib = library()
    _i32(rows, "rows")
    k = x.shape[1]
    m = rows.numel() if rows is not None else x.shape[0]
    n = w.shape[0]
    assert x.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
    assert w.shape[1] == k and w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    _check(lib.hfee_gemm_stream_norm(x.data_ptr(), _rows(x, "x"), _ptr(rows), norm_weight.data_ptr(), float(eps),
                                     int(add_unit), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                     _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _stream()), lib)


# Norming inside the streaming GEMM saves a launch, but every CTA then reads the float32 rows (twice
# the bytes of the normed bfloat16 rows, the same addresses from every SM at the same moment).
# Measured on B200 in the model: batch 1 gains (0.765 -> 0.737 ms per decode step), batch 8 loses
# (0.88 -> 0.92 ms); the break-even lies near three tokens.
FUSE_NORM_MAX_TOKENS = 2
FUSE_NORM_MAX_WIDTH = 2048      # one pass of the kernel that keeps the tokens in registers


def _norm_fusable(inp, w: torch.Tensor) -> bool:
    """True when ``inp`` (a lazily normed input, see parts/norm.py) can be normed inside the streaming GEMM."""
    if inp.n > FUSE_NORM_MAX_TOKENS:
        return False
    p = inp.fused_params()
    x = inp.source
    return (p is not None and inp.out_dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and inp.n <= 8 and x.shape[1] % 8 == 0 and x.shape[1] <= FUSE_NORM_MAX_WIDTH and _rows(x, "x") % 4 == 0
            and _rows(w, "w") % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and p[0].data_ptr() % 16 == 0)


def linear_normed(inp, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= norm(x) @ w.T where ``inp`` is a lazily normed input: the norm runs inside the
    product when a kernel that can do so fits, else ``inp`` is materialised first."""
    if isinstance(inp, torch.Tensor):
        linear(inp, w, out, accumulate)
    elif _norm_fusable(inp, w):
        weight, eps, add_unit = inp.fused_params()
        gemm_stream_norm(inp.source, weight, eps, w, out, EPI_ACCUM if accumulate else EPI_STORE, inp.rows, add_unit)
    else:
        linear(inp.tensor(), w, out, accumulate)


def linear_swiglu_normed(inp, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int, scratch: torch.Tensor) -> None:
    """:func:`linear_swiglu` on a lazily normed input."""
    if isinstance(inp, torch.Tensor):
        linear_swiglu(inp, w_gate_up, out, granule, scratch)
    elif granule == SWIGLU_GRANULE and w_gate_up.shape[0] % 8 == 0 and _norm_fusable(inp, w_gate_up):
        weight, eps, add_unit = inp.fused_params()
        gemm_stream_norm(inp.source, weight, eps, w_gate_up, out, EPI_SWIGLU, inp.rows, add_unit)
    else:
        linear_swiglu(inp.tensor(), w_gate_up, out, granule, scratch)


_SKINNY_WS: Optional[torch.Tensor] = None
SKINNY_WS_FLOATS = 4 << 20


def _skinny_workspace() -> torch.Tensor:
    """Float32 workspace for the partial tiles of K-split skinny products (made once, 16 MiB)."""
    global _SKINNY_WS
    if _SKINNY_WS is None:
        _SKINNY_WS = torch.empty(SKINNY_WS_FLOATS, dtype=torch.float32, device="cuda")
    return _SKINNY_WS


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 64 rows of ``a`` on tcgen05 with the operands swapped (weight
    rows on the 128-row side of the MMA) and K split among CTAs when weight tiles are few; TMA
    streams the weights through a deep shared-memory ring.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue in EPI_GATED else n)
    ws = _skinny_workspace()
    _check(lib.hfee_gemm_skinny(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, ws.data_ptr(), ws.numel(),
                                _status().data_ptr(), _stream()), lib)
    if lib.hfee_gemm_skinny_splits(m, n, k, ws.numel()) > 1:
        count_launches(1)


# The ring kernel (one CTA per SM, TMA boxes) against the register-streaming one, decode step of the
# benchmark model at batch 8: accumulating products (output and down projection) through the ring
# 0.873 -> 0.855 ms; all products through it 0.887 ms (gate/up and qkv, whose CTAs own several row
# tiles, are slower there); for one or two tokens the register kernel wins everywhere.
RING_MIN_TOKENS, RING_MAX_TOKENS = 3, 8
RING_EPILOGUES = (EPI_ACCUM,)
STREAM_BEST_TOKENS = 16      # up to here the register-streaming kernels win; above, the skinny tcgen05 kernel


def _small_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> None:
    m, n = a.shape[0], w.shape[0]
    if _ring_rule(m, n, a.shape[1], epilogue):
        gemm_ring(a, w, out, epilogue)
    elif m <= STREAM_BEST_TOKENS or not USE_TCGEN05:
        gemm_stream(a, w, out, epilogue)
    elif m > 32 and 64 * 128 <= n <= 256 * 128 and a.shape[1] <= 4096 and _tensor_core_ok(a, w) and (
            epilogue not in EPI_GATED or out.dtype == torch.bfloat16):
        # 64-256 narrow tiles of the large-tile kernel fill the SMs about once, and their epilogues are cheaper than the
        # swapped one: measured at 64 tokens, N = 16,384, K = 2,048: 16.3 us against 18.9 us
        gemm_tcgen05(a, w, out, epilogue)
    else:
        gemm_skinny(a, w, out, epilogue)


def _ring_rule(m: int, n: int, k: int, epilogue: int) -> bool:
    return (epilogue in RING_EPILOGUES and RING_MIN_TOKENS <= m <= RING_MAX_TOKENS and USE_TCGEN05
            and n <= 16 * sm_count() and ring_takes(m, n, k, epilogue))


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T, choosing the kernel for the dtype and the shape."""
    if _streamable(a, w):
        _small_gemm(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
    elif USE_TCGEN05 and _tensor_core_ok(a, w):
        gemm_tcgen05(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
    else:
        gemm_simt(a, w, out, accumulate)


SWIGLU_GRANULE = 4


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int,
                  scratch: torch.Tensor, activation: str = "silu") -> None:
    """out = act(a @ w_gate^T) * (a @ w_up^T) (``activation``: ``"silu"`` or ``"gelu_tanh"``) where ``w_gate_up`` holds the rows of both in groups
    of ``granule`` gate rows followed by ``granule`` up rows; ``scratch`` [m, 2*inner] holds the
    projection when it is not fused."""
    fusable = granule == SWIGLU_GRANULE and w_gate_up.shape[0] % 8 == 0
    epilogue = EPI_SWIGLU if activation == "silu" else EPI_GEGLU
    if fusable and _streamable(a, w_gate_up):
        _small_gemm(a, w_gate_up, out, epilogue)
    elif fusable and USE_TCGEN05 and _tensor_core_ok(a, w_gate_up) and out.dtype == torch.bfloat16:
        gemm_tcgen05(a, w_gate_up, out, epilogue)
    else:
        linear(a, w_gate_up, scratch)
        gated_act(scratch, out, activation, granule)


def linear_gated_normed(inp, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int, scratch: torch.Tensor,
                        activation: str) -> None:
    """:func:`linear_swiglu` with another gate activation (``"gelu_tanh"``): in the product's epilogue where a
    kernel with gated epilogues takes the shape, else through ``scratch`` [m, 2*inner] and :func:`gated_act`."""
    a = inp if isinstance(inp, torch.Tensor) else inp.tensor()
    linear_swiglu(a, w_gate_up, out, granule, scratch, activation)


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                   page_size: int, positions: torch.Tensor, slot_of_token: torch.Tensor, out: torch.Tensor,
                   heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal GQA over the paged cache, one warp per (token, head), float32 math."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = q.shape[0]
    assert q.shape[1] == heads * head_dim and out.shape == q.shape and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_attention_simt(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                   block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(),
                                   slot_of_token.data_ptr(), out.data_ptr(), _rows(out, "attention out"), n, heads,
                                   kv_heads, head_dim, float(scale), int(window or 0), _dt(q), _stream()), lib)


MAX_SPLITS = 32


def attention_splits(requests: int, kv_heads: int, max_context: int, sms: Optional[int] = None) -> int:
    """How many CTAs share the keys of one (request, kv head) in a decode step: about four CTAs
    per SM in all (measured alone at batch 8: 9 splits against 6 take 10.3 / 27.2 / 90.8 us against
    11.3 / 30.9 / 99.6 us at 2,048 / 8,192 / 32,768 keys; batch 12 at 8,192 keys: 6 against 4 take
    37.5 against 42.6 us), and at least four even when the batch alone would fill the GPU (shorter
    CTAs balance better and keep more loads in flight: at 2,048 keys, batch 32: 41.8 us unsplit,
    33.4 us with four), but at least two key blocks of 64 each.  With few (request, kv head) pairs,
    two CTAs per SM: those grids take the kernel variant with four key blocks in flight per CTA, of
    which the step's shared-memory carve-out holds one per SM (decode step of the benchmark model at
    batch 2 / 3 / 4 / 5 / 6: 0.742 / 0.777 / 0.786 / 0.802 / 0.817 ms against 0.755 / 0.798 / 0.809 /
    0.812 / 0.823 with four per SM; at batch 8: 0.857 against 0.838)."""
    pairs = max(1, requests * kv_heads)
    per_sm = 2 if pairs <= FEW_PAIRS else 4
    want = max(4, per_sm * (sms or sm_count()) // pairs)
    return max(1, min(MAX_SPLITS, want, max_context // 128))


FEW_PAIRS = 48


def attention_mma(q, k_pool, v_pool, block_table, page_size, cu_tokens, slots, context_before, out, n_tokens,
                  requests, max_new, heads, kv_heads, head_dim, scale, window=0, num_splits=1, scratch=None) -> None:
    """Flash attention over the paged cache on mma.sync tensor cores (bfloat16)."""
    lib = library()
    for t, what in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (slots, "slots"),
                    (context_before, "context_before")):
        _i32(t, what)
    assert q.dtype == k_pool.dtype == out.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    if num_splits > 1:
        need = n_tokens * heads * num_splits * (head_dim + 2)
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
    _check(lib.hfee_attention_mma(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                  block_table.data_ptr(), block_table.shape[1], page_size, cu_tokens.data_ptr(),
                                  slots.data_ptr(), context_before.data_ptr(), out.data_ptr(),
                                  _rows(out, "attention out"), n_tokens, requests, max_new, heads, kv_heads,
                                  head_dim, float(scale), int(window or 0), num_splits, _ptr(scratch), _stream()), lib)
    if num_splits > 1:
        count_launches(1)


USE_TC_ATTENTION = True


def attention_tc(q, k_pool, v_pool, block_table, page_size, cu_tokens, slots, context_before, out, n_tokens,
                 requests, max_new, heads, kv_heads, head_dim, scale, window=0) -> None:
    """Flash attention for prompt portions on tcgen05 (S, P and O in tensor memory, TMA-fed pages, one
    softmax thread per query row).  bfloat16, head size 64 or 128, pages of at least 64 tokens."""
    lib = library()
    for t, what in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (slots, "slots"),
                    (context_before, "context_before")):
        _i32(t, what)
    assert q.dtype == k_pool.dtype == out.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_attention_tc(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0],
                                 block_table.data_ptr(), block_table.shape[1], page_size, cu_tokens.data_ptr(),
                                 slots.data_ptr(), context_before.data_ptr(), out.data_ptr(),
                                 _rows(out, "attention out"), n_tokens, requests, max_new, heads, kv_heads, head_dim,
                                 float(scale), int(window or 0), _status().data_ptr(), _stream()), lib)


_TC_TAKES: dict = {}


def attention_tc_supports(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    key = (heads, kv_heads, head_dim, page_size)
    if key not in _TC_TAKES:
        _TC_TAKES[key] = bool(library().hfee_attention_tc_supports(*key))
    return _TC_TAKES[key]


def paged_attention(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                    head_dim, scale, window=0, step=None, scratch=None) -> None:
    """Attention over the cache, choosing the kernel for the dtype and the batch.  ``step`` gives
    the per-request layout (cu_tokens, slots, context_before, max_new, max_context) that the
    tensor-core kernel needs; without it, or in float32, the CUDA-core kernel runs."""
    group = heads // kv_heads
    if (step is not None and q.dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and group <= 64 and _rows(q, "q") % 8 == 0):
        if (USE_TC_ATTENTION and step.max_new * group > 16 and _rows(out, "out") % 8 == 0
                and attention_tc_supports(heads, kv_heads, head_dim, page_size)):
            attention_tc(q, k_pool, v_pool, block_table, page_size, step.cu_tokens, step.slots, step.context_before,
                         out, step.n, step.r, step.max_new, heads, kv_heads, head_dim, scale, window)
            return
        splits = 1
        if step.max_new * group <= 16 and scratch is not None:
            splits = getattr(step, "attention_splits", None) or attention_splits(
                step.r, kv_heads, getattr(step, "planning_context", step.max_context))
            if step.n * heads * splits * (head_dim + 2) > scratch.numel():
                splits = 1
        attention_mma(q, k_pool, v_pool, block_table, page_size, step.cu_tokens, step.slots, step.context_before,
                      out, step.n, step.r, step.max_new, heads, kv_heads, head_dim, scale, window, splits, scratch)
    else:
        attention_simt(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                       head_dim, scale, window)


# A decode step of one token per request can do the rotary kernel's work inside the attention
# kernel (one launch less per layer).
FUSE_ROPE_INTO_DECODE_ATTENTION = True


def decode_rope_fusable(step, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rope_dim: int,
                        qkv: torch.Tensor, scratch: Optional[torch.Tensor]) -> bool:
    """True when :func:`paged_attention_rope` takes this step: bfloat16, one new token per request,
    a group that fits the 16-row decode tile, rotary pieces of whole 16-byte units."""
    group = heads // kv_heads
    return (FUSE_ROPE_INTO_DECODE_ATTENTION and step is not None and dtype == torch.bfloat16
            and getattr(step, "max_new", 0) == 1 and group <= 16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and rope_dim % 16 == 0 and _rows(qkv, "qkv") % 8 == 0 and qkv.data_ptr() % 16 == 0)


def paged_attention_rope(qkv, cs, rope_dim, interleaved, write_cache, k_pool, v_pool, block_table, page_size, out,
                         heads, kv_heads, head_dim, scale, window, step, scratch) -> None:
    """Rotary + cache write + attention of a decode step in one kernel (plus the combine kernel when
    the keys are split): ``qkv`` rows are [q heads | k heads | v heads] ([q heads] when
    ``write_cache`` is false), ``cs`` the (cos, sin) table of the step or None."""
    lib = library()
    for t, what in ((block_table, "block_table"), (step.cu_tokens, "cu_tokens"), (step.slots, "slots"),
                    (step.context_before, "context_before")):
        _i32(t, what)
    assert qkv.dtype == k_pool.dtype == out.dtype == torch.bfloat16 and step.n == step.r
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == step.n * rope_dim)
    splits = 1
    if scratch is not None:
        splits = getattr(step, "attention_splits", None) or attention_splits(
            step.r, kv_heads, getattr(step, "planning_context", step.max_context))
        if step.n * heads * splits * (head_dim + 2) > scratch.numel():
            splits = 1
    _check(lib.hfee_attention_mma_rope(qkv.data_ptr(), _rows(qkv, "qkv"), _ptr(cs), rope_dim, int(interleaved),
                                       int(write_cache), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                       block_table.shape[1], page_size, step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                       step.context_before.data_ptr(), out.data_ptr(), _rows(out, "attention out"),
                                       step.n, step.r, heads, kv_heads, head_dim, float(scale), int(window or 0), splits,
                                       _ptr(scratch) if splits > 1 else None, _stream()), lib)
    if splits > 1:
        count_launches(1)


# ---------------------------------------------------------------------------- mechanisms beside softmax attention
WEIGHTS_SOFTMAX, WEIGHTS_SIGMOID = 0, 1
ACTIVATIONS = {"none": 0, "silu": 1}
GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def attention_simt_masked(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                          head_dim, scale, window=0, chunk=0, weights=WEIGHTS_SOFTMAX, head_scale=None, head_bias=None,
                          gate=None) -> None:
    """:func:`attention_simt` with its options: ``chunk`` > 0 lets a query see only keys of its own block of
    ``chunk`` positions (counted from position 0 of the request); ``weights`` = WEIGHTS_SIGMOID replaces the
    softmax by unnormalised weights sigmoid(score * head_scale[h] + head_bias[h]); ``gate`` [n, heads * head_dim]
    multiplies the output by sigmoid(gate) element by element.  float32 arithmetic in both dtypes."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = q.shape[0]
    assert q.shape[1] == heads * head_dim and out.shape == q.shape and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    for t in (head_scale, head_bias):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads)
    assert gate is None or (gate.dtype == q.dtype and gate.shape == q.shape)
    _check(lib.hfee_attention_simt_masked(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                          block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(),
                                          slot_of_token.data_ptr(), out.data_ptr(), _rows(out, "attention out"), n, heads,
                                          kv_heads, head_dim, float(scale), int(window or 0), int(chunk or 0), int(weights),
                                          _ptr(head_scale), _ptr(head_bias), _ptr(gate),
                                          _rows(gate, "gate") if gate is not None else 0, _dt(q), _stream()), lib)


def short_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor,
               write_state: bool = True) -> None:
    """out[t] = x[t] + sum_j weight[:, j] * x[t - taps + 1 + j] per request of the step, inputs in front of the
    step's tokens taken from ``state`` [slots, taps - 1, width] (float32), which then takes the request's last
    taps - 1 inputs.  ``x`` is float32 [n, width]; ``out`` may be float32 or bfloat16."""
    lib = library()
    n, width = x.shape
    taps = weight.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32 and weight.is_contiguous()
    assert weight.shape[0] == width and state.dtype == torch.float32 and state.is_contiguous()
    assert tuple(state.shape[1:]) == (taps - 1, width) and out.shape == x.shape
    _check(lib.hfee_short_conv(x.data_ptr(), weight.data_ptr(), state.data_ptr(), step.cu_tokens.data_ptr(),
                               step.slots.data_ptr(), out.data_ptr(), _rows(out, "conv out"), _dt(out), step.r,
                               step.max_new, width, taps, int(write_state), _stream()), lib)
    if lib.hfee_short_conv_launches(step.max_new, taps, int(write_state)) > 1:
        count_launches(1)


# Prompt portions of at least this many tokens (the longest of the step) take the chunked kernels.
LINEAR_ATTENTION_CHUNKED_MIN = 8


def linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                     step, out: torch.Tensor, heads: int, dim: int, vdim: int, activation: str = "none",
                     write_state: bool = True, workspace: Optional[torch.Tensor] = None,
                     chunked: Optional[bool] = None, tensor_cores: bool = True) -> None:
    """Linear attention with a decay per head over the step's tokens, continuing each request's float32 state
    ``state`` [slots, heads, dim, vdim]: S <- decay_h S + k v^T, o = S^T q.  ``q``, ``k``, ``v`` are column
    slices of one projection buffer (same row stride); ``activation`` is applied to them on the way in;
    ``out`` is float32 [n, heads * vdim].  Steps with a portion of several tokens take the chunked kernels
    when ``workspace`` (float32, see :func:`linear_attention_workspace`) is given, else the token-by-token one;
    the chunked kernels run on the tensor cores for bfloat16 activations and key sizes that are multiples of 16
    (``tensor_cores=False``: on the CUDA cores)."""
    lib = library()
    n = q.shape[0]
    assert q.dtype == k.dtype == v.dtype and q.stride(0) == k.stride(0) == v.stride(0) and q.stride(1) == 1
    assert q.shape[1] == k.shape[1] == heads * dim and v.shape[1] == heads * vdim
    assert decay.dtype == torch.float32 and decay.numel() == heads and state.dtype == torch.float32 and state.is_contiguous()
    assert tuple(state.shape[1:]) == (heads, dim, vdim) and out.dtype == torch.float32 and out.shape == (n, heads * vdim)
    act = ACTIVATIONS[activation]
    if chunked is None:
        chunked = workspace is not None and step.max_new >= LINEAR_ATTENTION_CHUNKED_MIN
    if chunked:
        need = lib.hfee_linear_attention_chunked_workspace(step.r, step.n, heads, dim, vdim)
        assert workspace is not None and workspace.dtype == torch.float32 and workspace.numel() >= need, (need,)
        _check(lib.hfee_linear_attention_chunked(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), _dt(q),
                                                 decay.data_ptr(), state.data_ptr(), step.cu_tokens.data_ptr(),
                                                 step.slots.data_ptr(), out.data_ptr(), _rows(out, "out"),
                                                 workspace.data_ptr(), workspace.numel(), step.r, step.n, heads,
                                                 dim, vdim, act, int(write_state), int(tensor_cores), _stream()), lib)
        count_launches(2)
        return
    _check(lib.hfee_linear_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), _dt(q), decay.data_ptr(),
                                     state.data_ptr(), step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(),
                                     _rows(out, "out"), step.r, heads, dim, vdim, act, int(write_state), _stream()), lib)


def linear_attention_workspace(requests: int, tokens: int, heads: int, dim: int, vdim: int) -> int:
    """Floats of workspace the chunked linear attention needs for a step of ``tokens`` tokens in ``requests`` requests."""
    return int(library().hfee_linear_attention_chunked_workspace(requests, tokens, heads, dim, vdim))


USE_SIGMOID_MMA = True
_SIGMOID_MMA_TAKES: dict = {}


def sigmoid_mma_supports(heads: int, kv_heads: int, head_dim: int) -> bool:
    key = (heads, kv_heads, head_dim)
    if key not in _SIGMOID_MMA_TAKES:
        _SIGMOID_MMA_TAKES[key] = bool(library().hfee_attention_sigmoid_mma_supports(*key))
    return _SIGMOID_MMA_TAKES[key]


def sigmoid_attention(q, k_pool, v_pool, block_table, page_size, step, out, heads, kv_heads, head_dim, scale, window=0,
                      chunk=0, head_scale=None, head_bias=None, gate=None) -> None:
    """Attention with unnormalised sigmoid weights over the cache, choosing the kernel for the dtype and the
    sizes: bfloat16 with a head size and a group the tensor-core kernel is built for runs there (prompt portions
    and decode steps alike), everything else on the CUDA cores in float32."""
    if USE_SIGMOID_MMA and q.dtype == torch.bfloat16 and sigmoid_mma_supports(heads, kv_heads, head_dim) and (
            _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0 and _rows(out, "out") % 2 == 0 and (gate is None or (_rows(gate, "gate") % 2 == 0
                                                                                     and gate.data_ptr() % 4 == 0))):
        lib = library()
        for t, what in ((block_table, "block_table"), (step.cu_tokens, "cu_tokens"), (step.slots, "slots"),
                        (step.context_before, "context_before")):
            _i32(t, what)
        assert k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim) and q.shape == out.shape == (step.n, heads * head_dim)
        _check(lib.hfee_attention_sigmoid_mma(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                              block_table.data_ptr(), block_table.shape[1], page_size,
                                              step.cu_tokens.data_ptr(), step.slots.data_ptr(), step.context_before.data_ptr(),
                                              out.data_ptr(), _rows(out, "out"), step.n, step.r, heads, kv_heads, head_dim,
                                              float(scale), int(window or 0), int(chunk or 0), _ptr(head_scale),
                                              _ptr(head_bias), _ptr(gate), _rows(gate, "gate") if gate is not None else 0,
                                              _stream()), lib)
        return
    attention_simt_masked(q, k_pool, v_pool, block_table, page_size, step.positions, step.slot_of_token, out, heads,
                          kv_heads, head_dim, scale, window, chunk, WEIGHTS_SIGMOID, head_scale, head_bias, gate)


# ---------------------------------------------------------------------------- independent key and value sizes, latents, the delta rule
GATE_NONE, GATE_ELEMENT, GATE_PER_HEAD = 0, 1, 2
HEAD_GATE_ACTIVATIONS = {"sigmoid": 0, "silu": 1}
UNARY_ACTIVATIONS = {"relu2": 0}


def attention_simt_general(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                           head_dim, value_dim, scale, window=0, chunk=0, gate=None, gate_mode=GATE_NONE) -> None:
    """Softmax attention over the paged cache on the CUDA cores in float32 arithmetic with a value size of its
    own: ``v_pool`` is [pages, kv_heads, page_size, value_dim], or None when the values are the leading
    ``value_dim`` dimensions of the cached keys.  ``gate`` multiplies the output by its sigmoid: one number per
    output element (GATE_ELEMENT, [n, heads * value_dim]) or per head (GATE_PER_HEAD, [n, heads])."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = q.shape[0]
    assert q.shape[1] == heads * head_dim and tuple(out.shape) == (n, heads * value_dim) and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    if v_pool is not None:
        assert v_pool.is_contiguous() and v_pool.dtype == q.dtype and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim)
    assert (gate is None) == (gate_mode == GATE_NONE) and (gate is None or gate.dtype == q.dtype)
    _check(lib.hfee_attention_simt_general(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), _ptr(v_pool), block_table.data_ptr(),
                                           block_table.shape[1], page_size, positions.data_ptr(), slot_of_token.data_ptr(),
                                           out.data_ptr(), _rows(out, "attention out"), n, heads, kv_heads, head_dim,
                                           value_dim, int(v_pool is None), float(scale), int(window or 0), int(chunk or 0),
                                           WEIGHTS_SOFTMAX, None, None, _ptr(gate),
                                           _rows(gate, "gate") if gate is not None else 0, int(gate_mode), _dt(q), _stream()), lib)


def attention_simt_distance(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                            head_dim, value_dim, scale, r1, r2, out_scale=1.0, window=0) -> None:
    """:func:`attention_simt_general` with a penalty on distance: ``r1[h] * ln(1 + r2[h] * (i - j))`` is taken off
    the score of key j for query i of head h before the softmax (``r1``, ``r2`` float32 per head); the output is
    multiplied by ``out_scale``."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = q.shape[0]
    assert q.shape[1] == heads * head_dim and tuple(out.shape) == (n, heads * value_dim) and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    assert v_pool.is_contiguous() and v_pool.dtype == q.dtype and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim)
    for r in (r1, r2):
        assert r.dtype == torch.float32 and r.is_contiguous() and r.numel() == heads
    _check(lib.hfee_attention_simt_distance(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                            block_table.shape[1], page_size, positions.data_ptr(), slot_of_token.data_ptr(),
                                            out.data_ptr(), _rows(out, "attention out"), n, heads, kv_heads, head_dim,
                                            value_dim, 0, float(scale), int(window or 0), 0, WEIGHTS_SOFTMAX, None, None, None, 0,
                                            GATE_NONE, r1.data_ptr(), r2.data_ptr(), float(out_scale), _dt(q), _stream()), lib)


DISTANCE_ATTENTION_ON_TENSOR_CORES = True
_DISTANCE_TILE: dict = {}


def distance_attention_tile(head_dim: int, value_dim: int) -> int:
    """Tile size (floats per partial output) of the tensor-core kernel for these key and value sizes; 0: it does not
    take them."""
    key = (head_dim, value_dim)
    if key not in _DISTANCE_TILE:
        _DISTANCE_TILE[key] = int(library().hfee_attention_mma_distance_tile(head_dim, value_dim))
    return _DISTANCE_TILE[key]


def distance_attention(q, k_pool, v_pool, block_table, page_size, step, out, heads, kv_heads, head_dim, value_dim, scale, r1, r2,
                       out_scale=1.0, window=0, scratch=None) -> None:
    """Causal grouped-query softmax attention over the paged cache whose scores lose ``r1[h] * ln(1 + r2[h] * distance)``,
    choosing the kernel for the dtype and the step: bfloat16 with key and value sizes that are multiples of 8 (up to 256)
    runs on the tensor cores (prompt portions, decode steps with their keys split among CTAs when ``scratch`` is given,
    and mixtures), everything else on the CUDA cores in float32 arithmetic."""
    group = heads // kv_heads
    tile = distance_attention_tile(head_dim, value_dim) if (DISTANCE_ATTENTION_ON_TENSOR_CORES and q.dtype == torch.bfloat16) else 0
    if not (tile and group <= 64 and _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0 and _rows(out, "out") % 4 == 0
            and out.data_ptr() % 8 == 0):
        attention_simt_distance(q, k_pool, v_pool, block_table, page_size, step.positions, step.slot_of_token, out, heads, kv_heads,
                                head_dim, value_dim, scale, r1, r2, out_scale, window)
        return
    lib = library()
    for t, what in ((block_table, "block_table"), (step.cu_tokens, "cu_tokens"), (step.slots, "slots"),
                    (step.context_before, "context_before")):
        _i32(t, what)
    assert k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim) and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim)
    assert q.shape[1] == heads * head_dim and tuple(out.shape) == (step.n, heads * value_dim)
    for r in (r1, r2):
        assert r.dtype == torch.float32 and r.is_contiguous() and r.numel() == heads
    splits = 1
    if step.max_new * group <= 16 and scratch is not None:
        splits = getattr(step, "attention_splits", None) or attention_splits(
            step.r, kv_heads, getattr(step, "planning_context", step.max_context))
        if step.n * heads * splits * (tile + 2) > scratch.numel():
            splits = 1
    _check(lib.hfee_attention_mma_distance(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                           block_table.shape[1], page_size, step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                           step.context_before.data_ptr(), out.data_ptr(), _rows(out, "attention out"), step.n,
                                           step.r, step.max_new, heads, kv_heads, head_dim, value_dim, float(scale), r1.data_ptr(),
                                           r2.data_ptr(), float(out_scale), int(window or 0), splits,
                                           _ptr(scratch) if splits > 1 else None, _stream()), lib)
    if splits > 1:
        count_launches(1)


# The grouped-query kernels on the tensor cores take bfloat16 queries and keys and round the softmax weights to
# bfloat16 for the product with the values; the CUDA-core kernel keeps scores and weights in float32.
GATED_ATTENTION_ON_TENSOR_CORES = True


def softmax_attention_on_tensor_cores(q: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                                      value_dim: int, page_size: int, step) -> bool:
    """True when :func:`paged_attention` runs this step on the tensor cores: bfloat16, values of the keys' size,
    and sizes those kernels are built for."""
    group = heads // kv_heads
    if not (GATED_ATTENTION_ON_TENSOR_CORES and q.dtype == torch.bfloat16 and head_dim == value_dim and step is not None
            and head_dim % 16 == 0 and 16 <= head_dim <= 256 and group <= 64 and _rows(q, "q") % 8 == 0):
        return False
    return True


def latent_attention(q: torch.Tensor, k_pool: torch.Tensor, block_table: torch.Tensor, page_size: int, step,
                     out: torch.Tensor, heads: int, cached_dim: int, value_dim: int, scale: float, window: int = 0) -> None:
    """Softmax attention of ``heads`` query heads over ONE cached vector per token (``k_pool`` [pages, 1, page_size,
    cached_dim]) whose leading ``value_dim`` dimensions are also the values: ``out`` [n, heads * value_dim].
    bfloat16 with sizes the tensor-core kernel takes runs there (prompt portions and decode steps alike),
    everything else on the CUDA cores in float32."""
    if (USE_LATENT_MMA and q.dtype == torch.bfloat16 and latent_mma_supports(heads, cached_dim, value_dim)
            and _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0 and _rows(out, "out") % 2 == 0 and out.data_ptr() % 4 == 0):
        lib = library()
        for t, what in ((block_table, "block_table"), (step.cu_tokens, "cu_tokens"), (step.slots, "slots"),
                        (step.context_before, "context_before")):
            _i32(t, what)
        assert k_pool.dtype == out.dtype == torch.bfloat16 and k_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (1, page_size, cached_dim)
        assert tuple(q.shape) == (step.n, heads * cached_dim) and tuple(out.shape) == (step.n, heads * value_dim)
        _check(lib.hfee_latent_attention_mma(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), block_table.data_ptr(),
                                             block_table.shape[1], page_size, step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                             step.context_before.data_ptr(), out.data_ptr(), _rows(out, "out"), step.r,
                                             step.max_new, heads, cached_dim, value_dim, float(scale), int(window or 0),
                                             _stream()), lib)
        return
    attention_simt_general(q, k_pool, None, block_table, page_size, step.positions, step.slot_of_token, out, heads, 1,
                           cached_dim, value_dim, scale, window)


USE_LATENT_MMA = True
_LATENT_MMA_TAKES: dict = {}


def latent_mma_supports(heads: int, cached_dim: int, value_dim: int) -> bool:
    key = (heads, cached_dim, value_dim)
    if key not in _LATENT_MMA_TAKES:
        _LATENT_MMA_TAKES[key] = bool(library().hfee_latent_attention_mma_supports(*key))
    return _LATENT_MMA_TAKES[key]


def linear_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(a @ w.T) for an activation of :data:`UNARY_ACTIVATIONS`: in the product's epilogue where the
    large-tile tcgen05 kernels take the shape, else by a pass of its own over the result."""
    if (activation == "relu2" and USE_TCGEN05 and not _streamable(a, w) and _tensor_core_ok(a, w)
            and out.dtype == torch.bfloat16):
        gemm_tcgen05(a, w, out, EPI_RELU2)
        return
    linear(a, w, out)
    unary_act(out, out, activation)


def rope_norm_cache(src: torch.Tensor, cs: Optional[torch.Tensor], rope_dim: int, norm_eps: Optional[float],
                    positions: torch.Tensor, slot_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                    q=None, k=None, v=None) -> None:
    """Per head of a row of ``src``: rotate ``rope_dim`` dimensions (dimension i with i + rope_dim/2) by the step's
    (cos, sin) table ``cs``, then divide the head by its root mean square (``norm_eps`` None: no norm), and store.
    ``q`` = (heads, src_off, src_stride, len, rope_off, out, dst_off, dst_stride): queries into the buffer ``out``;
    ``k`` = (kv_heads, src_off, src_stride, len, rope_off, pool, dst_off): keys into their cache page at ``dst_off``
    within the cached vector; ``v`` = (src_off, src_stride, len, pool): values copied as they are.  Any may be None."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = src.shape[0]
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * rope_dim)
    qh, qso, qss, ql, qro, qout, qdo, qds = q if q is not None else (0, 0, 0, 0, 0, None, 0, 0)
    kh, kso, kss, kl, kro, kpool, kdo = k if k is not None else (0, 0, 0, 0, 0, None, 0)
    vso, vss, vl, vpool = v if v is not None else (0, 0, 0, None)
    for t in (qout, kpool, vpool):
        assert t is None or t.dtype == src.dtype
    assert kpool is None or (kpool.is_contiguous() and kpool.shape[1] == kh and kpool.shape[2] == page_size)
    assert vpool is None or (vpool.is_contiguous() and kpool is not None and vpool.shape[1] == kh and vpool.shape[2] == page_size)
    _check(lib.hfee_rope_norm_cache(src.data_ptr(), _rows(src, "src"), _dt(src), n, _ptr(cs), int(rope_dim) if cs is not None else 0,
                                    -1.0 if norm_eps is None else float(norm_eps), positions.data_ptr(), slot_of_token.data_ptr(),
                                    qh, qso, qss, ql, qro, _ptr(qout), _rows(qout, "q out") if qout is not None else 0, qdo, qds,
                                    kh, kso, kss, kl, kro, _ptr(kpool), kpool.shape[3] if kpool is not None else 0, kdo,
                                    vso, vss, vl, _ptr(vpool), vpool.shape[3] if vpool is not None else 0,
                                    block_table.data_ptr(), block_table.shape[1], page_size, _stream()), lib)


def latent_norm_rope_cache(proj: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int,
                           q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float, cs: torch.Tensor,
                           positions: torch.Tensor, slot_of_token: torch.Tensor, cq_out: torch.Tensor,
                           k_pool: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int) -> None:
    """The down-projections of a latent attention, per token: ``proj[:, q_off : q_off + q_rank]`` RMS-normed with
    ``q_weight`` into ``cq_out``; ``proj[:, kv_off : kv_off + kv_rank]`` RMS-normed with ``kv_weight`` into the leading
    dimensions of the token's cached vector and the ``rot_dim`` columns behind it, rotated, into the rest
    (``k_pool`` [pages, 1, page_size, kv_rank + rot_dim]; None: only the query latent)."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = proj.shape[0]
    assert q_weight.dtype == kv_weight.dtype == torch.float32 and q_weight.numel() == q_rank and kv_weight.numel() == kv_rank
    assert cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * rot_dim and cq_out.dtype == proj.dtype
    if k_pool is not None:
        assert k_pool.dtype == proj.dtype and k_pool.is_contiguous() and tuple(k_pool.shape[1:]) == (1, page_size, kv_rank + rot_dim)
    _check(lib.hfee_latent_norm_rope_cache(proj.data_ptr(), _rows(proj, "proj"), _dt(proj), n, q_off, q_rank, kv_off, kv_rank,
                                           rot_dim, q_weight.data_ptr(), kv_weight.data_ptr(), float(eps), cs.data_ptr(),
                                           positions.data_ptr(), slot_of_token.data_ptr(), cq_out.data_ptr(),
                                           _rows(cq_out, "cq_out"), _ptr(k_pool), block_table.data_ptr(), block_table.shape[1],
                                           page_size, _stream()), lib)


def head_linear(x: torch.Tensor, in_off: int, in_stride: int, w: torch.Tensor, out: torch.Tensor, out_off: int,
                out_stride: int, gate: Optional[torch.Tensor] = None) -> None:
    """out[i, out_off + h * out_stride + o] = sum_k w[h, o, k] * x[i, in_off + h * in_stride + k], times
    sigmoid(gate[i, h]) if ``gate`` [n, heads] is given.  ``w`` is [heads, n_out, n_in]."""
    lib = library()
    heads, n_out, n_in = w.shape
    n = x.shape[0]
    assert w.is_contiguous() and x.dtype == w.dtype == out.dtype and out.shape[0] == n
    assert in_off + (heads - 1) * in_stride + n_in <= x.shape[1] and out_off + (heads - 1) * out_stride + n_out <= out.shape[1]
    assert gate is None or (gate.dtype == x.dtype and gate.shape == (n, heads))
    _check(lib.hfee_head_linear(x.data_ptr(), _rows(x, "x"), in_off, in_stride, w.data_ptr(), out.data_ptr(), _rows(out, "out"),
                                out_off, out_stride, n, heads, n_in, n_out, _ptr(gate),
                                _rows(gate, "gate") if gate is not None else 0, _dt(x), _stream()), lib)


def conv_act(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor, activation: str = "silu",
             write_state: bool = True, bias: Optional[torch.Tensor] = None) -> None:
    """out[t, c] = act(bias[c] + sum_j weight[c, j] * x[t - taps + 1 + j, c]) per request of the step (``bias`` None: 0), inputs in front of the
    step's tokens taken from ``state`` [slots, taps - 1, width] (float32), which then takes the request's last
    taps - 1 inputs.  ``x`` and ``out`` are [n, width] views (any row stride) of the activations' dtype."""
    lib = library()
    n, width = x.shape
    taps = weight.shape[1]
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == width
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, width)
    assert out.shape == x.shape and out.dtype == x.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == width)
    _check(lib.hfee_conv_act(x.data_ptr(), _rows(x, "conv in"), _dt(x), weight.data_ptr(), _ptr(bias), state.data_ptr(),
                             step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), _rows(out, "conv out"), step.r,
                             step.max_new, width, taps, ACTIVATIONS[activation], int(write_state), _stream()), lib)
    if lib.hfee_conv_act_launches(step.max_new, taps, int(write_state)) > 1:
        count_launches(1)


def delta_rule(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, ba: torch.Tensor, b_off: int, a_off: int,
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor, heads: int,
               qk_heads: int, dim: int, vdim: int, write_state: bool = True, workspace: Optional[torch.Tensor] = None) -> None:
    """The gated delta rule over the step's tokens, continuing each request's float32 state ``state``
    [slots, heads, dim, vdim]: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with q and k made unit
    vectors per head first (q also times dim^-1/2), beta = sigmoid(b) and g = exp(-exp(a_log) softplus(a + dt_bias)).
    ``qkv`` rows hold the queries and keys of ``qk_heads`` heads and the values of ``heads`` heads at the given
    column offsets, ``ba`` rows one b and one a per head.  ``out`` is float32 [n, heads * vdim].  With ``workspace``
    (float32, see :func:`delta_rule_workspace`) a step that has a portion of several tokens runs as two kernels: what
    does not depend on the state for all tiles of 16 tokens at once, then the walk over each request's tiles."""
    lib = library()
    n = qkv.shape[0]
    assert qkv.dtype == ba.dtype and ba.shape[0] == n and out.dtype == torch.float32 and tuple(out.shape) == (n, heads * vdim)
    assert a_log.dtype == dt_bias.dtype == torch.float32 and a_log.numel() == dt_bias.numel() == heads
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim)
    assert max(q_off, k_off) + qk_heads * dim <= qkv.shape[1] and v_off + heads * vdim <= qkv.shape[1]
    assert max(b_off, a_off) + heads <= ba.shape[1]
    assert workspace is None or (workspace.dtype == torch.float32 and workspace.is_contiguous())
    _check(lib.hfee_delta_rule(qkv.data_ptr(), _rows(qkv, "qkv"), q_off, k_off, v_off, ba.data_ptr(), _rows(ba, "ba"), b_off,
                               a_off, _dt(qkv), a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(),
                               step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), _rows(out, "out"), step.r,
                               heads, qk_heads, dim, vdim, int(write_state), step.n, step.max_new, _ptr(workspace),
                               workspace.numel() if workspace is not None else 0, _stream()), lib)
    if workspace is not None and step.max_new > 1:
        count_launches(1)


def delta_rule_workspace(requests: int, tokens: int, heads: int, qk_heads: int, dim: int) -> int:
    """Floats of workspace the two-kernel delta rule needs for a step of ``tokens`` tokens in ``requests`` requests."""
    return int(library().hfee_delta_rule_workspace(requests, tokens, heads, qk_heads, dim))


def head_norm_gate(x: torch.Tensor, weight: torch.Tensor, eps: float, gate: torch.Tensor, out: torch.Tensor, heads: int,
                   head_dim: int, activation: str = "sigmoid") -> None:
    """Per (row, head): out = x / sqrt(mean over the head of x^2 + eps) * weight[d] * act(gate), ``weight`` [head_dim]
    shared by the heads, ``act`` sigmoid or SiLU.  ``x`` is float32; ``gate`` and ``out`` share a dtype."""
    lib = library()
    n = x.shape[0]
    assert x.dtype == torch.float32 and gate.dtype == out.dtype and tuple(gate.shape) == tuple(x.shape) == tuple(out.shape) == (n, heads * head_dim)
    assert weight.dtype == torch.float32 and weight.numel() == head_dim
    _check(lib.hfee_head_norm_gate(x.data_ptr(), _rows(x, "x"), weight.data_ptr(), float(eps), gate.data_ptr(), _rows(gate, "gate"),
                                   out.data_ptr(), _rows(out, "out"), n, heads, head_dim, HEAD_GATE_ACTIVATIONS[activation],
                                   _dt(out), _stream()), lib)


def unary_act(x: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(x) element by element; ``activation``: ``"relu2"`` (the square of relu).  ``out`` may be ``x``."""
    lib = library()
    assert x.shape == out.shape and x.dtype == out.dtype and x.dim() == 2
    _check(lib.hfee_unary_act(x.data_ptr(), _rows(x, "x"), out.data_ptr(), _rows(out, "out"), x.shape[0], x.shape[1],
                              UNARY_ACTIVATIONS[activation], _dt(x), _stream()), lib)


def head_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, head_dim: int) -> None:
    """x[i, h * head_dim + d] *= sigmoid(gate[i, h]) in place."""
    lib = library()
    n = x.shape[0]
    assert x.shape[1] == heads * head_dim and gate.dtype == x.dtype and tuple(gate.shape) == (n, heads)
    _check(lib.hfee_head_gate(x.data_ptr(), _rows(x, "x"), gate.data_ptr(), _rows(gate, "gate"), n, heads, head_dim, _dt(x),
                              _stream()), lib)


def rmsnorm_add(y: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, eps: float, add_unit: bool = False,
                cast_out: Optional[torch.Tensor] = None) -> None:
    """residual += y * rsqrt(mean(y^2) + eps) * weight, all float32.  With ``cast_out`` the new residual rows
    are also written there in its dtype (what the next matrix product reads)."""
    lib = library()
    assert y.dtype == residual.dtype == weight.dtype == torch.float32 and residual.is_contiguous()
    n, width = residual.shape
    assert y.shape == residual.shape and weight.numel() == width
    assert cast_out is None or cast_out.shape == residual.shape
    _check(lib.hfee_rmsnorm_add(y.data_ptr(), _rows(y, "y"), weight.data_ptr(), residual.data_ptr(), n, width,
                                float(eps), int(add_unit), _ptr(cast_out),
                                _rows(cast_out, "cast_out") if cast_out is not None else 0,
                                _dt(cast_out) if cast_out is not None else 0, _stream()), lib)


RMSNORM_ADD_NORM_MAX_WIDTH = 12288          # the row is kept in shared memory


def rmsnorm_add_norm(y: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, eps: float, weight2: torch.Tensor,
                     eps2: float, out: torch.Tensor, add_unit: bool = False, add_unit2: bool = False) -> None:
    """residual += y * rsqrt(mean(y^2) + eps) * weight, then out = residual * rsqrt(mean(residual^2) + eps2) * weight2
    in ``out``'s dtype: the norm on a sublayer's output and the norm in front of the next sublayer in one kernel."""
    lib = library()
    assert y.dtype == residual.dtype == weight.dtype == weight2.dtype == torch.float32 and residual.is_contiguous()
    n, width = residual.shape
    assert y.shape == residual.shape == out.shape and weight.numel() == weight2.numel() == width
    _check(lib.hfee_rmsnorm_add_norm(y.data_ptr(), _rows(y, "y"), weight.data_ptr(), residual.data_ptr(), n, width, float(eps),
                                     int(add_unit), weight2.data_ptr(), float(eps2), int(add_unit2), out.data_ptr(),
                                     _rows(out, "out"), _dt(out), _stream()), lib)


def norm_gate(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out = (x * rsqrt(mean(x^2) + eps) * weight) * sigmoid(gate); without ``weight`` only the gate.
    ``x`` is float32; ``gate`` and ``out`` share a dtype."""
    lib = library()
    n, width = x.shape
    assert x.dtype == torch.float32 and gate.dtype == out.dtype and gate.shape == x.shape == out.shape
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == width)
    _check(lib.hfee_norm_gate(x.data_ptr(), _rows(x, "x"), _ptr(weight), float(eps), gate.data_ptr(), _rows(gate, "gate"),
                              out.data_ptr(), _rows(out, "out"), n, width, _dt(out), _stream()), lib)


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, granule: Optional[int] = None) -> None:
    """out[i, c] = act(gate) * up with the column layout of :func:`swiglu`; ``activation`` is ``"silu"`` or
    ``"gelu_tanh"`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))."""
    lib = library()
    n, inter = out.shape
    assert gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype
    _check(lib.hfee_gated_act(gate_up.data_ptr(), _rows(gate_up, "gate_up"), out.data_ptr(), _rows(out, "out"), n, inter,
                              int(granule or inter), GATE_ACTIVATIONS[activation], _dt(out), _stream()), lib)


def scale_(x: torch.Tensor, alpha: float) -> None:
    """x *= alpha (float32, rows contiguous)."""
    lib = library()
    assert x.dtype == torch.float32 and x.dim() == 2
    _check(lib.hfee_scale_f32(x.data_ptr(), _rows(x, "x"), x.shape[0], x.shape[1], float(alpha), _stream()), lib)


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32, contiguous) rounded to ``out``'s dtype."""
    lib = library()
    assert x.dtype == torch.float32 and x.is_contiguous() and out.shape == x.shape
    _check(lib.hfee_cast_rows(x.data_ptr(), out.data_ptr(), _rows(out, "out"), x.shape[0], x.shape[1], _dt(out), _stream()), lib)


# ---------------------------------------------------------------------------- scaled and averaged residual streams, capped logits
def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, base: float = 10000.0) -> None:
    """x[t, 2i] += sin(p_t * base^(-2i/width)), x[t, 2i+1] += cos of the same angle (float32 rows, float64 angles)."""
    lib = library()
    _i32(positions, "positions")
    assert x.dtype == torch.float32 and x.is_contiguous() and positions.numel() == x.shape[0]
    _check(lib.hfee_add_sinusoid(x.data_ptr(), positions.data_ptr(), x.shape[0], x.shape[1], float(base), _stream()), lib)


def softcap_(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place (float32 rows)."""
    lib = library()
    assert x.dtype == torch.float32 and x.dim() == 2
    _check(lib.hfee_softcap(x.data_ptr(), _rows(x, "x"), x.shape[0], x.shape[1], float(cap), _stream()), lib)


CLAMPED_SWISH_ALPHA = 1.702


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float = CLAMPED_SWISH_ALPHA,
                granule: Optional[int] = None, shift: float = 1.0) -> None:
    """out = g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit); column layout
    of :func:`swiglu`.  An infinite limit, alpha = 1 and shift = 0 give silu(gate) * up."""
    lib = library()
    n, inner = out.shape
    assert gate_up.shape[1] == 2 * inner and gate_up.dtype == out.dtype
    _check(lib.hfee_clamped_glu(gate_up.data_ptr(), _rows(gate_up, "gate_up"), out.data_ptr(), _rows(out, "out"), n, inner,
                                int(granule or inner), float(limit), float(alpha), float(shift), _dt(out), _stream()), lib)


def scaled_add_norm(y: torch.Tensor, m: float, residual: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """residual += m * y (both float32), then out = residual / sqrt(mean(residual^2) + eps) * weight in ``out``'s dtype."""
    lib = library()
    n, width = residual.shape
    assert y.dtype == residual.dtype == weight.dtype == torch.float32 and y.is_contiguous() and residual.is_contiguous()
    assert y.shape == residual.shape and tuple(out.shape) == (n, width) and weight.numel() == width
    _check(lib.hfee_scaled_add_norm(y.data_ptr(), float(m), residual.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(),
                                    _rows(out, "out"), n, width, _dt(out), _stream()), lib)


def scaled_add(y: torch.Tensor, m: float, residual: torch.Tensor) -> None:
    """residual += m * y (both float32)."""
    lib = library()
    n, width = residual.shape
    assert y.dtype == residual.dtype == torch.float32 and y.is_contiguous() and residual.is_contiguous() and y.shape == residual.shape
    _check(lib.hfee_scaled_add_norm(y.data_ptr(), float(m), residual.data_ptr(), None, 0.0, None, 0, n, width, _DT[torch.float32],
                                    _stream()), lib)


def depth_average(residual: torch.Tensor, y: Optional[torch.Tensor], m: float, history: torch.Tensor, weights: torch.Tensor,
                  index: int) -> None:
    """r = residual + m * y (``y`` None: r = residual); history[index + 1, :n] = r;
    residual = sum_(j <= index) weights[j] * history[j, :n] + weights[index + 1] * r.  ``history`` is
    [entries, rows, width] float32 with entries >= index + 2."""
    lib = library()
    n, width = residual.shape
    assert residual.dtype == history.dtype == weights.dtype == torch.float32 and residual.is_contiguous() and history.is_contiguous()
    assert history.shape[0] >= index + 2 and history.shape[1] >= n and history.shape[2] == width and weights.numel() == index + 2
    assert y is None or (y.dtype == torch.float32 and y.is_contiguous() and y.shape == residual.shape)
    _check(lib.hfee_depth_average(residual.data_ptr(), _ptr(y), float(m), history.data_ptr(), history.stride(0), weights.data_ptr(),
                                  int(index), n, width, _stream()), lib)


# ---------------------------------------------------------------------------- elementwise recurrences
def mingru(proj: torch.Tensor, z_off: int, x_off: int, g_off: int, z_bias: torch.Tensor, x_bias: torch.Tensor, state: torch.Tensor,
           step, out: torch.Tensor, channels: int, write_state: bool = True) -> None:
    """z = sigmoid(proj_z + z_bias), u = proj_x + x_bias, c = u + 1/2 where u >= 0 else sigmoid(u);
    S_t = (1 - z) S_(t-1) + z c per channel from ``state`` [slots, channels] (float32, renewed);
    out = S_t * silu(proj_g) in the activations' dtype."""
    lib = library()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == channels
    assert out.dtype == proj.dtype and out.shape[1] == channels and max(z_off, x_off, g_off) + channels <= proj.shape[1]
    _check(lib.hfee_mingru(proj.data_ptr(), _rows(proj, "proj"), z_off, x_off, g_off, z_bias.data_ptr(), x_bias.data_ptr(),
                           state.data_ptr(), step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), _rows(out, "out"),
                           step.r, step.max_new, channels, int(write_state), _dt(proj), _stream()), lib)


def selective_scan(x: torch.Tensor, dt_proj: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, z: torch.Tensor,
                   a_log: torch.Tensor, d_skip: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor,
                   out_scale: float = 1.0, write_state: bool = True) -> None:
    """dt = softplus(dt_proj + dt_bias), A = -exp(a_log); S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;
    y_c = sum_n S[c, n] C_n + d_skip_c x_c; out = y * silu(z) * out_scale.  ``state`` [slots, channels, n] float32
    is read and renewed; B and C are columns of ``bc``; ``dt_proj`` is float32."""
    lib = library()
    n, channels = x.shape
    n_state = a_log.shape[1]
    assert dt_proj.dtype == torch.float32 and tuple(dt_proj.shape) == (n, channels)
    assert a_log.dtype == torch.float32 and a_log.is_contiguous() and a_log.shape[0] == channels
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (channels, n_state)
    assert z.dtype == x.dtype == bc.dtype == out.dtype and z.shape == x.shape == out.shape
    assert max(b_off, c_off) + n_state <= bc.shape[1]
    _check(lib.hfee_selective_scan(x.data_ptr(), _rows(x, "x"), dt_proj.data_ptr(), _rows(dt_proj, "dt"), bc.data_ptr(), _rows(bc, "bc"),
                                   b_off, c_off, z.data_ptr(), _rows(z, "z"), a_log.data_ptr(), d_skip.data_ptr(), dt_bias.data_ptr(),
                                   state.data_ptr(), step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), _rows(out, "out"),
                                   step.r, step.max_new, channels, n_state, float(out_scale), int(write_state), _dt(x), _stream()), lib)


# ---------------------------------------------------------------------------- routed experts
def moe_tile_rows() -> int:
    return int(library().hfee_moe_tile_rows())


def moe_max_tiles(pairs: int, experts: int) -> int:
    """Tiles a plan of ``pairs`` (token, choice) pairs over ``experts`` experts can need."""
    return pairs // moe_tile_rows() + experts + 1


def moe_route(logits: torch.Tensor, top: int, scale: float, choice: torch.Tensor, weight: torch.Tensor) -> None:
    """Per row of ``logits`` [n, experts] (float32): softmax over all experts, the ``top`` largest (ties: the lower
    expert) into ``choice`` [n, top] int32, their scores times ``scale`` into ``weight`` [n, top] float32."""
    lib = library()
    n, experts = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and weight.dtype == torch.float32
    _i32(choice, "choice")
    assert tuple(choice.shape) == (n, top) and tuple(weight.shape) == (n, top) and weight.is_contiguous()
    _check(lib.hfee_moe_route(logits.data_ptr(), n, experts, top, float(scale), choice.data_ptr(), weight.data_ptr(), _stream()), lib)


def moe_route_grouped(logits: torch.Tensor, experts: int, top: int, groups: int, keep: int, scale: float, choice: torch.Tensor,
                      weight: torch.Tensor) -> None:
    """Per row of ``logits`` (float32; the first ``experts`` columns): scores sigmoid(logit); the experts form ``groups``
    equal groups of neighbours, a group's score is the sum of its two largest scores, and only experts of the ``keep`` best
    groups can be chosen; the ``top`` largest of those (ties: the lower expert) into ``choice`` [n, top] int32, their
    scores divided by their sum and times ``scale`` into ``weight`` [n, top] float32."""
    lib = library()
    n = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= experts and weight.dtype == torch.float32
    _i32(choice, "choice")
    assert tuple(choice.shape) == (n, top) and tuple(weight.shape) == (n, top) and weight.is_contiguous()
    _check(lib.hfee_moe_route_grouped(logits.data_ptr(), logits.stride(0), n, experts, top, groups, keep, float(scale),
                                      choice.data_ptr(), weight.data_ptr(), _stream()), lib)


def moe_plan(choice: torch.Tensor, experts: int, offsets: torch.Tensor, order: torch.Tensor, tile_expert: torch.Tensor,
             tile_row: torch.Tensor) -> None:
    """Order the (token, choice) pairs by expert: ``offsets`` [experts + 1], ``order`` [pairs] (pair index at each
    place), and the tiles of places (``tile_expert`` -1 = unused)."""
    lib = library()
    for t in (choice, offsets, order, tile_expert, tile_row):
        _i32(t, "moe plan")
    pairs = choice.numel()
    assert offsets.numel() == experts + 1 and order.numel() >= pairs and tile_row.numel() == tile_expert.numel()
    _check(lib.hfee_moe_plan(choice.data_ptr(), pairs, experts, offsets.data_ptr(), order.data_ptr(), tile_expert.data_ptr(),
                             tile_row.data_ptr(), tile_expert.numel(), _stream()), lib)


def moe_experts(x: torch.Tensor, top: int, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, limit: float,
                offsets: torch.Tensor, order: torch.Tensor, tile_expert: torch.Tensor, tile_row: torch.Tensor,
                hidden: torch.Tensor, pair_out: torch.Tensor, alpha: float = CLAMPED_SWISH_ALPHA, shift: float = 1.0) -> None:
    """For every (token, chosen expert e) pair: pair_out[pair] = W_down[e] act(W_gate[e] x, W_up[e] x) (float32), with the
    clamped gated activation of :func:`clamped_glu`.  ``w_gate``, ``w_up``: [experts, inner, width]; ``w_down``:
    [experts, width, inner]; ``hidden`` [pairs, inner] is scratch in the activations' dtype."""
    lib = library()
    n, width = x.shape
    experts, inner = w_gate.shape[0], w_gate.shape[1]
    pairs = n * top
    tiles = min(tile_expert.numel(), moe_max_tiles(pairs, experts))
    # gate and up may be the two halves of one [experts, 2 * inner, width] tensor: each expert's matrix dense, one stride
    assert w_down.is_contiguous() and w_gate.stride() == w_up.stride() and w_gate.stride()[1:] == (width, 1)
    assert tuple(w_up.shape) == (experts, inner, width) and tuple(w_down.shape) == (experts, width, inner)
    assert x.dtype == w_gate.dtype == w_up.dtype == w_down.dtype == hidden.dtype
    assert hidden.shape[0] >= pairs and hidden.shape[1] == inner
    assert pair_out.dtype == torch.float32 and pair_out.is_contiguous() and pair_out.shape[0] >= pairs and pair_out.shape[1] == width
    _check(lib.hfee_moe_gate_up(x.data_ptr(), _rows(x, "x"), top, w_gate.data_ptr(), w_up.data_ptr(), w_gate.stride(0), inner, width,
                                offsets.data_ptr(),
                                order.data_ptr(), tile_expert.data_ptr(), tile_row.data_ptr(), hidden.data_ptr(),
                                _rows(hidden, "hidden"), float(limit), float(alpha), float(shift), tiles, _dt(x), _stream()), lib)
    _check(lib.hfee_moe_down(hidden.data_ptr(), _rows(hidden, "hidden"), top, w_down.data_ptr(), inner, width, offsets.data_ptr(),
                             order.data_ptr(), tile_expert.data_ptr(), tile_row.data_ptr(), pair_out.data_ptr(), tiles, _dt(x),
                             _stream()), lib)


def moe_combine(pair_out: torch.Tensor, weight: torch.Tensor, y: torch.Tensor, accumulate: bool,
                place: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
                extra_gate: Optional[torch.Tensor] = None) -> None:
    """y[t] (+)= sum_k weight[t, k] * pair_out[row of pair t * top + k] (float32); the row is ``place[pair]``, or the
    pair's index without ``place``.  ``extra`` [n, width] float32 is one more term per token, times
    ``sigmoid(extra_gate[t])`` when ``extra_gate`` (a float32 column, any row stride) is given."""
    lib = library()
    n, top = weight.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape[0] == n and pair_out.shape[1] == y.shape[1]
    assert pair_out.dtype == torch.float32 and pair_out.is_contiguous()
    if place is not None:
        _i32(place, "place")
        assert place.numel() >= n * top
    if extra is not None:
        assert extra.dtype == torch.float32 and extra.is_contiguous() and tuple(extra.shape) == tuple(y.shape)
    if extra_gate is not None:
        assert extra is not None and extra_gate.dtype == torch.float32 and extra_gate.shape[0] == n
    _check(lib.hfee_moe_combine_extra(pair_out.data_ptr(), weight.data_ptr(), _ptr(place), n, top, y.data_ptr(), y.shape[1],
                                      int(accumulate), _ptr(extra), _ptr(extra_gate),
                                      extra_gate.stride(0) if extra_gate is not None else 0, _stream()), lib)


GROUPED_TILE_ROWS = 128         # rows of a tile of the grouped product


def moe_tiles_grouped(pairs: int, experts: int) -> int:
    """Tiles of GROUPED_TILE_ROWS rows that ``pairs`` pairs over ``experts`` experts can need when every expert starts at
    a tile's border: an expert with c pairs fills c // 128 tiles and at most one more, and no more experts have pairs
    than there are pairs."""
    return pairs // GROUPED_TILE_ROWS + min(experts, pairs)


def moe_experts_grouped_ok(x_dtype: torch.dtype, width: int, inner: int) -> bool:
    """Whether :func:`moe_experts_grouped` takes these: bfloat16, rows of whole 16-byte pieces."""
    return x_dtype == torch.bfloat16 and width % 8 == 0 and inner % 8 == 0


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, out: torch.Tensor,
                         clamped: Optional[tuple] = None) -> None:
    """out[rows of tile i] = a[rows of tile i] @ w[tile_group[i]].T for tiles of GROUPED_TILE_ROWS rows; tiles whose
    group is negative are left alone, and so is everything behind the first of them (the tiles in use come first).
    ``a`` [tiles * 128, k] bfloat16, ``w`` [groups, n, k] bfloat16 contiguous,
    ``out`` [tiles * 128, n] bfloat16 or float32.  ``tile_group`` is read on the device.  With ``clamped`` = (limit,
    alpha) every group's rows come in runs of [4 gate | 4 up] and ``out`` [tiles * 128, n / 2] bfloat16 receives
    :func:`clamped_glu` of the product, applied to the float32 accumulator."""
    lib = library()
    m, k = a.shape
    groups, n = w.shape[0], w.shape[1]
    _i32(tile_group, "tile_group")
    assert w.shape[2] == k and w.is_contiguous() and a.dtype == w.dtype == torch.bfloat16
    assert m % GROUPED_TILE_ROWS == 0 and tile_group.numel() >= m // GROUPED_TILE_ROWS
    assert tuple(out.shape) == (m, n // 2 if clamped else n)
    limit, alpha, shift = (tuple(clamped) + (1.0,))[:3] if clamped else (0.0, 0.0, 0.0)
    _check(lib.hfee_gemm_tcgen05_grouped(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), k, out.data_ptr(), _rows(out, "gemm out"),
                                         _dt(out), m, n, k, groups, tile_group.data_ptr(), int(clamped is not None), float(limit),
                                         float(alpha), float(shift), _status().data_ptr(), _stream()), lib)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, granule: int = 4) -> torch.Tensor:
    """[..., inner, k] twice -> [..., 2 * inner, k] with the rows in runs of ``granule`` gate rows and ``granule`` up rows,
    the layout of the gated epilogues."""
    inner = gate.shape[-2]
    lead = gate.shape[:-2]
    w = torch.stack([gate.reshape(*lead, inner // granule, granule, -1), up.reshape(*lead, inner // granule, granule, -1)], dim=-3)
    return w.reshape(*lead, 2 * inner, -1).contiguous()


CLAMPED_PAIR_MIN_TOKENS = 65


def linear_clamped_glu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int, scratch: torch.Tensor,
                       limit: float, alpha: float = 1.702, shift: float = 1.0) -> None:
    """out = :func:`clamped_glu` of ``a @ w_gate_up^T`` (rows of ``w_gate_up`` in runs of ``granule`` gate and ``granule`` up
    rows): in the epilogue of the paired tcgen05 product for prompt portions in bfloat16, else through ``scratch``
    [m, 2 * inner]."""
    m, k = a.shape
    n = w_gate_up.shape[0]
    if (granule == SWIGLU_GRANULE and n % 8 == 0 and m >= CLAMPED_PAIR_MIN_TOKENS and USE_TCGEN05 and USE_PAIRS
            and _tensor_core_ok(a, w_gate_up) and out.dtype == torch.bfloat16):
        lib = library()
        _check(lib.hfee_gemm_tcgen05_pair_clamped(a.data_ptr(), _rows(a, "gemm a"), w_gate_up.data_ptr(), _rows(w_gate_up, "gemm w"),
                                                  out.data_ptr(), _rows(out, "gemm out"), m, n, k, float(limit), float(alpha),
                                                  float(shift), _status().data_ptr(), _stream()), lib)
        return
    linear(a, w_gate_up, scratch)
    clamped_glu(scratch, out, limit, alpha, granule, shift)


def moe_experts_grouped(x: torch.Tensor, top: int, choice: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, limit: float,
                        place: torch.Tensor, row_pair: torch.Tensor, tile_group: torch.Tensor, rows_in: torch.Tensor,
                        gate_up: torch.Tensor, hidden: torch.Tensor, rows_out: torch.Tensor,
                        alpha: float = CLAMPED_SWISH_ALPHA, shift: float = 1.0) -> None:
    """The experts' two products on the tensor cores: rows_out[place[pair]] = W_down[e] act(W_gate[e] x, W_up[e] x) for every
    (token, chosen expert e) pair, float32.  ``w_gate_up`` [experts, 2 * inner, width] holds each expert's gate rows, then
    its up rows; ``w_down`` [experts, width, inner].  Scratch, all of ``tiles * 128`` rows with ``tiles =
    moe_tiles_grouped(pairs, experts)``: ``rows_in`` [., width], ``gate_up`` [., 2 * inner], ``hidden`` [., inner]
    (bfloat16), ``rows_out`` [., width] float32; ``place`` [pairs], ``row_pair`` [tiles * 128], ``tile_group`` [tiles].
    With ``gate_up`` None each expert's rows of ``w_gate_up`` come in runs of [4 gate | 4 up] (:func:`interleave_gate_up`)
    and the activation runs in the first product's epilogue."""
    lib = library()
    n, width = x.shape
    experts, inner = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    pairs = n * top
    tiles = moe_tiles_grouped(pairs, experts)
    rows = tiles * GROUPED_TILE_ROWS
    for t in (choice, place, row_pair, tile_group):
        _i32(t, "moe plan")
    assert choice.numel() == pairs and place.numel() >= pairs and row_pair.numel() >= rows and tile_group.numel() >= tiles
    assert rows_in.shape[0] >= rows and (gate_up is None or gate_up.shape[0] >= rows) and hidden.shape[0] >= rows and rows_out.shape[0] >= rows
    _check(lib.hfee_moe_plan_tiles(choice.data_ptr(), pairs, experts, GROUPED_TILE_ROWS, place.data_ptr(), row_pair.data_ptr(),
                                   tile_group.data_ptr(), tiles, _stream()), lib)
    _check(lib.hfee_moe_gather_rows(x.data_ptr(), _rows(x, "x"), top, row_pair.data_ptr(), tile_group.data_ptr(), GROUPED_TILE_ROWS,
                                    rows_in.data_ptr(), _rows(rows_in, "rows_in"), width, tiles, _stream()), lib)
    if gate_up is None:         # the activation in the first product's epilogue
        gemm_tcgen05_grouped(rows_in[:rows], w_gate_up, tile_group, hidden[:rows], clamped=(limit, alpha, shift))
    else:
        gemm_tcgen05_grouped(rows_in[:rows], w_gate_up, tile_group, gate_up[:rows])
        clamped_glu(gate_up[:rows], hidden[:rows], limit, alpha, shift=shift)
    gemm_tcgen05_grouped(hidden[:rows], w_down, tile_group, rows_out[:rows])


def qk_norm_rope_cache(qk: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cs: Optional[torch.Tensor], rope_dim: int, positions: torch.Tensor, slot_of_token: torch.Tensor,
                       q_out: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       block_table: torch.Tensor, page_size: int, heads: int, kv_heads: int, head_dim: int,
                       v_offset: int = -1) -> None:
    """Rows of ``qk`` are [query projection | key projection].  Each is RMS-normed as a whole (all heads at
    once, weights ``q_weight`` / ``k_weight``; None = no norm), then the first ``rope_dim`` dimensions of every
    head are rotated (dimension i with i + rope_dim/2) by the step's (cos, sin) table ``cs``.  Queries go to
    ``q_out``, keys to their cache page, and the value page (if given) takes the key projection as it came
    (``v_offset`` < 0) or the ``kv_heads * head_dim`` columns of the row that start at ``v_offset``."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = qk.shape[0]
    want = (heads + kv_heads) * head_dim if k_pool is not None else heads * head_dim
    assert qk.shape[1] >= max(want, v_offset + kv_heads * head_dim) and q_out.dtype == qk.dtype and q_out.shape == (n, heads * head_dim)
    if k_pool is not None:
        assert k_pool.dtype == qk.dtype and k_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
        assert v_pool is None or (v_pool.dtype == qk.dtype and v_pool.is_contiguous() and v_pool.shape == k_pool.shape)
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * rope_dim)
    _check(lib.hfee_qk_norm_rope_cache(qk.data_ptr(), _rows(qk, "qk"), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cs),
                                       int(rope_dim) if cs is not None else 0, positions.data_ptr(), slot_of_token.data_ptr(),
                                       q_out.data_ptr(), _rows(q_out, "q_out"), _ptr(k_pool), _ptr(v_pool),
                                       block_table.data_ptr(), block_table.shape[1], page_size, n, heads, kv_heads,
                                       head_dim, int(v_offset), _dt(qk), _stream()), lib)


# ---------------------------------------------------------------------------- bigram embedding, layer norm, biases
def embed_bigram(table: torch.Tensor, pairs: torch.Tensor, step, last_token: torch.Tensor, out: torch.Tensor, buckets: int,
                 mul_prev: int, mul_cur: int) -> None:
    """out[i] = table[token_i] + pairs[(previous token * mul_prev + token_i * mul_cur) mod buckets] as float32; a request's
    first token takes row ``buckets``.  The token in front of a portion's first token is ``last_token[slot]`` (int32 per
    request slot), which is then set to the last token each request brought in this step."""
    lib = library()
    n, width = out.shape
    feedback = getattr(step, "feedback", None)
    _i32(step.token_ids, "tokens"); _i32(last_token, "last_token"); _i32(feedback, "feedback")
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and pairs.is_contiguous()
    assert table.dtype == pairs.dtype and tuple(pairs.shape) == (buckets + 1, width) and table.shape[1] == width
    _check(lib.hfee_embed_bigram(table.data_ptr(), pairs.data_ptr(), _dt(table), step.token_ids.data_ptr(), step.positions.data_ptr(),
                                 step.slot_of_token.data_ptr(), _ptr(feedback), last_token.data_ptr(), out.data_ptr(), n, width,
                                 table.shape[0], int(buckets), int(mul_prev), int(mul_cur), _stream()), lib)
    _check(lib.hfee_remember_tokens(step.token_ids.data_ptr(), step.slot_of_token.data_ptr(), _ptr(feedback),
                                    step.cu_tokens.data_ptr(), step.slots.data_ptr(), step.r, last_token.data_ptr(), _stream()), lib)


def layernorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
              residual_add: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x[rows[r] or r] - mean) / sqrt(variance + eps) * weight in float32 arithmetic (no bias).  With
    ``residual_add`` (float32, like ``x``) the row is ``x + residual_add`` and that sum is stored back to ``x``."""
    lib = library()
    _i32(rows, "layernorm rows")
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == x.shape[1]
    assert residual_add is None or (residual_add.dtype == torch.float32 and residual_add.is_contiguous()
                                    and residual_add.shape == x.shape and rows is None)
    n, width = out.shape
    _check(lib.hfee_layernorm(x.data_ptr(), _ptr(residual_add), weight.data_ptr(), _ptr(rows), out.data_ptr(), _rows(out, "out"),
                              _dt(out), n, width, float(eps), _stream()), lib)


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[r, c] += bias[c] (float32)."""
    lib = library()
    assert x.dtype == torch.float32 and bias.dtype == torch.float32 and bias.numel() == x.shape[1]
    _check(lib.hfee_add_bias(x.data_ptr(), _rows(x, "x"), bias.data_ptr(), x.shape[0], x.shape[1], _stream()), lib)


def attention_prepare(src: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, key_dim: int,
                      value_dim: int, step, q_out: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                      block_table: torch.Tensor, page_size: int, cs: Optional[torch.Tensor] = None, rope_dim: int = 0,
                      interleaved: bool = False, biases=(None, None, None), norm_weights=(None, None), eps: float = 0.0) -> None:
    """One token's [q | k | v] projection on its way to the score kernel: ``biases`` = (q, k, v) float32 per column (each may
    be None), ``norm_weights`` = (q, k) weights of an RMS norm over the whole query / key projection (None: no norm),
    then the rotation of the first ``rope_dim`` dimensions of every head by the step's (cos, sin) table ``cs``, pairing
    (i, i + rope_dim/2) or, ``interleaved``, (2i, 2i + 1).  Queries to ``q_out``, keys and values to their pages (pools None:
    queries only)."""
    lib = library()
    n = src.shape[0]
    _i32(block_table, "block_table")
    for t in biases + norm_weights:
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * rope_dim)
    assert q_out.dtype == src.dtype and q_out.shape[1] == heads * key_dim
    if k_pool is not None:
        assert k_pool.dtype == v_pool.dtype == src.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, key_dim) and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim)
    _check(lib.hfee_attention_prepare(src.data_ptr(), _rows(src, "src"), _dt(src), n, q_off, k_off, v_off, _ptr(biases[0]),
                                      _ptr(biases[1]), _ptr(biases[2]), _ptr(norm_weights[0]), _ptr(norm_weights[1]), float(eps),
                                      _ptr(cs), int(rope_dim) if cs is not None else 0, int(interleaved), step.positions.data_ptr(),
                                      step.slot_of_token.data_ptr(), q_out.data_ptr(), _rows(q_out, "q_out"), _ptr(k_pool),
                                      _ptr(v_pool), block_table.data_ptr(), block_table.shape[1], page_size, heads, kv_heads,
                                      key_dim, value_dim, _stream()), lib)


SOFTMAX_ATTENTION_ON_TENSOR_CORES = True


def softmax_attention(q, k_pool, v_pool, block_table, page_size, step, out, heads, kv_heads, head_dim, value_dim, scale,
                      window=0, sink=None, out_scale=1.0, scratch=None) -> None:
    """Causal grouped-query softmax attention over the paged cache with key and value sizes of their own, an optional
    window, an optional ``sink`` (float32 per query head: the denominator also holds exp(sink[h]), a term without key or
    value) and the output times ``out_scale``.  bfloat16 with key and value sizes that are multiples of 8 (up to 256) runs
    on the tensor cores (prompt portions, decode steps with their keys split among CTAs when ``scratch`` is given, and
    mixtures), everything else on the CUDA cores in float32 arithmetic."""
    lib = library()
    group = heads // kv_heads
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == heads)
    assert q.shape[1] == heads * head_dim and tuple(out.shape) == (step.n, heads * value_dim) and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and v_pool.dtype == q.dtype
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim) and tuple(v_pool.shape[1:]) == (kv_heads, page_size, value_dim)
    _i32(block_table, "block_table")
    tile = distance_attention_tile(head_dim, value_dim) if (SOFTMAX_ATTENTION_ON_TENSOR_CORES and q.dtype == torch.bfloat16) else 0
    if not (tile and group <= 64 and _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0 and _rows(out, "out") % 4 == 0
            and out.data_ptr() % 8 == 0):
        _check(lib.hfee_attention_simt_sink(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                            block_table.shape[1], page_size, step.positions.data_ptr(), step.slot_of_token.data_ptr(),
                                            out.data_ptr(), _rows(out, "attention out"), step.n, heads, kv_heads, head_dim,
                                            value_dim, 0, float(scale), int(window or 0), 0, WEIGHTS_SOFTMAX, None, None, None, 0,
                                            GATE_NONE, None, None, float(out_scale), _ptr(sink), _dt(q), _stream()), lib)
        return
    splits = 1
    if step.max_new * group <= 16 and scratch is not None:
        splits = getattr(step, "attention_splits", None) or attention_splits(
            step.r, kv_heads, getattr(step, "planning_context", step.max_context))
        if step.n * heads * splits * (tile + 2) > scratch.numel():
            splits = 1
    _check(lib.hfee_attention_mma_general(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                          block_table.shape[1], page_size, step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                          step.context_before.data_ptr(), out.data_ptr(), _rows(out, "attention out"), step.n,
                                          step.r, step.max_new, heads, kv_heads, head_dim, value_dim, float(scale), None, None,
                                          _ptr(sink), float(out_scale), int(window or 0), splits,
                                          _ptr(scratch) if splits > 1 else None, _stream()), lib)
    if splits > 1:
        count_launches(1)


RECURRENCE_CHANNEL_DECAY, RECURRENCE_EXP_GATES = 0, 1
RECURRENCE_CHUNKED_MIN = 65        # from this many new tokens of one request on, runs of 64 tokens work side by side


def gated_recurrence_workspace(requests: int, tokens: int, heads: int, dim: int, vdim: int) -> int:
    """Floats of workspace :func:`gated_recurrence` wants for steps of at most ``tokens`` tokens of ``requests`` requests."""
    return int(library().hfee_gated_recurrence_workspace(requests, tokens, heads, dim, vdim))


def gated_recurrence(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pre: torch.Tensor, bias: Optional[torch.Tensor],
                     p0: float, q_scale: float, state: torch.Tensor, step, out: torch.Tensor, heads: int, dim: int, vdim: int,
                     write_state: bool = True, norm_state: Optional[torch.Tensor] = None,
                     max_state: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> None:
    """Linear attention with a gated float32 matrix state per (request slot, head), token after token.
    RECURRENCE_CHANNEL_DECAY: S = diag(a) S + k v^T with a = sigmoid(pre + bias)^p0 per key channel (``pre`` [n, heads * dim]
    float32, ``p0`` = 1 / tau), o = S^T q.  RECURRENCE_EXP_GATES: ``pre`` [n, 2 * heads] float32 holds the input and forget
    gates' pre-activations x_i, x_f; i = p0 tanh(x_i / p0), f = logsigmoid(p0 tanh(x_f / p0)), m' = max(f + m, i),
    S = e^(f + m - m') S + e^(i - m') k v^T, n likewise with k alone, o = S^T q / (max(|n . q|, e^(-m')) + 1e-6), with
    ``norm_state`` [slots, heads, dim] and ``max_state`` [slots, heads].  ``q`` (times ``q_scale``), ``k``, ``v`` are
    column slices of one buffer; ``state`` [slots, heads, dim, vdim]; ``out`` [n, heads * vdim] float32.  With ``workspace``
    (float32, :func:`gated_recurrence_workspace`) and a request that brings RECURRENCE_CHUNKED_MIN tokens or more, runs of 64
    tokens are walked side by side (the same recurrence in another association); with the channel decay that path
    overwrites ``pre`` with the decays."""
    lib = library()
    ld = _rows(q, "q")
    assert _rows(k, "k") == ld and _rows(v, "v") == ld and q.dtype == k.dtype == v.dtype
    assert q.shape[1] == heads * dim and k.shape[1] == heads * dim and v.shape[1] == heads * vdim
    assert pre.dtype == torch.float32 and pre.stride(1) == 1 and out.dtype == torch.float32 and out.shape[1] == heads * vdim
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous())
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim)
    for t, shape in ((norm_state, (heads, dim)), (max_state, (heads,))):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape[1:]) == shape)
    if workspace is not None and step.max_new >= RECURRENCE_CHUNKED_MIN:
        assert workspace.dtype == torch.float32 and workspace.is_contiguous()
        _check(lib.hfee_gated_recurrence_chunked(int(mode), q.data_ptr(), k.data_ptr(), v.data_ptr(), ld, _dt(q), pre.data_ptr(),
                                                 pre.stride(0), _ptr(bias), float(p0), float(q_scale), state.data_ptr(),
                                                 _ptr(norm_state), _ptr(max_state), step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                                 out.data_ptr(), _rows(out, "out"), step.r, step.n, heads, dim, vdim,
                                                 int(write_state), workspace.data_ptr(), workspace.numel(), _stream()), lib)
        count_launches(2 + int(mode == RECURRENCE_EXP_GATES))
        return
    _check(lib.hfee_gated_recurrence(int(mode), q.data_ptr(), k.data_ptr(), v.data_ptr(), ld, _dt(q), pre.data_ptr(), pre.stride(0),
                                     _ptr(bias), float(p0), float(q_scale), state.data_ptr(), _ptr(norm_state), _ptr(max_state),
                                     step.cu_tokens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), _rows(out, "out"), step.r,
                                     heads, dim, vdim, int(write_state), _stream()), lib)


def head_norm_gate_scaled(x: torch.Tensor, weight: torch.Tensor, eps: float, gate: torch.Tensor, out: torch.Tensor, heads: int,
                          head_dim: int, activation: str = "sigmoid", out_scale: float = 1.0) -> None:
    """:func:`head_norm_gate` with the output times ``out_scale`` and a weight that is either [head_dim], shared by the
    heads, or [heads * head_dim]."""
    lib = library()
    n = x.shape[0]
    assert x.dtype == torch.float32 and gate.dtype == out.dtype and tuple(gate.shape) == tuple(x.shape) == tuple(out.shape) == (n, heads * head_dim)
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() in (head_dim, heads * head_dim)
    per_head = weight.numel() == heads * head_dim and heads > 1
    _check(lib.hfee_head_norm_gate_scaled(x.data_ptr(), _rows(x, "x"), weight.data_ptr(), int(per_head), float(eps), gate.data_ptr(),
                                          _rows(gate, "gate"), out.data_ptr(), _rows(out, "out"), n, heads, head_dim,
                                          HEAD_GATE_ACTIVATIONS[activation], float(out_scale), _dt(out), _stream()), lib)



def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
           feedback: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or no temperatures are given),
    else a draw from softmax(logits[r] / temperature[r]) using uniform[r] in [0, 1): the inverse CDF
    over the tokens in the fixed order of the kernel (chunks of 2,048 ids; in a chunk the ids
    t, t + 256, ... of t = 0..255 in turn).  With ``slots`` and ``feedback`` the choice is also stored
    in ``feedback[slots[r]]``."""
    lib = library()
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.is_contiguous()
    _i32(slots, "slots"); _i32(feedback, "feedback")
    assert (slots is None) == (feedback is None)
    m, v = logits.shape
    if temperature is not None:
        assert temperature.dtype == torch.float32 and uniform.dtype == torch.float64
    global _SAMPLE_SCRATCH
    need = m * -(-v // CHAIN_CHUNK) * 2
    if _SAMPLE_SCRATCH is None or _SAMPLE_SCRATCH.numel() < need:
        _SAMPLE_SCRATCH = torch.empty(max(need, 64 * 64 * 2), dtype=torch.float64, device=logits.device)
    _check(lib.hfee_sample(logits.data_ptr(), _rows(logits, "logits"), m, v, _ptr(temperature), _ptr(uniform),
                           _SAMPLE_SCRATCH.data_ptr(), _SAMPLE_SCRATCH.numel(), out.data_ptr(), _ptr(slots),
                           _ptr(feedback), _stream()), lib)
    count_launches(1)


_SAMPLE_SCRATCH: Optional[torch.Tensor] = None


CHAIN_MAX_K = 64            # largest top-k the device chain takes
CHAIN_HISTORY = 256         # tokens of recent history kept per request slot for the repeat penalty
CHAIN_CHUNK = 2048
CHAIN_MAX_VOCAB = 128 * CHAIN_CHUNK     # the chain kernels look at no more chunks than this; larger vocabularies take the host chain


def chain_scratch_floats(rows: int, vocab: int) -> int:
    return rows * -(-vocab // CHAIN_CHUNK) * CHAIN_MAX_K * 2


def sample_chain(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
                 slots: Optional[torch.Tensor] = None, feedback: Optional[torch.Tensor] = None,
                 history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
                 penalise: bool = False) -> None:
    """The reference's sampling chain on the device: repeat penalty over the request's recent tokens
    (``history`` [slots, cap] rings with ``history_len`` [slots] tokens appended so far), the top-k
    logits (1 <= k <= CHAIN_MAX_K; greedy rows are k = 1), float64 probabilities, top-p and min-p
    cuts, the draw.  ``params`` [m, 8] float64 per row: temperature, top_k, top_p, min_p, repeat
    penalty, repeat_last_n, uniform number, unused.  ``logits`` is changed in place where a row
    penalises; the choice is appended to the request's ring and stored in ``feedback[slots[r]]``."""
    lib = library()
    m, v = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.is_contiguous()
    assert params.dtype == torch.float64 and params.is_contiguous() and tuple(params.shape) == (m, 8)
    assert scratch.dtype == torch.float32 and scratch.numel() >= chain_scratch_floats(m, v)
    _i32(slots, "slots"); _i32(feedback, "feedback"); _i32(history, "history"); _i32(history_len, "history_len")
    cap = history.shape[1] if history is not None else 0
    _check(lib.hfee_sample_chain(logits.data_ptr(), _rows(logits, "logits"), m, v, params.data_ptr(), _ptr(slots),
                                 _ptr(history), cap, _ptr(history_len), int(penalise), scratch.data_ptr(),
                                 scratch.numel(), out.data_ptr(), _ptr(feedback), _stream()), lib)
    count_launches(2 if penalise else 1)


ARGMAX_CHUNKS = 64


def argmax(logits: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, slots: Optional[torch.Tensor] = None,
           feedback: Optional[torch.Tensor] = None) -> None:
    """out[r] = index of the first maximum of logits[r]; ``scratch`` holds rows * ARGMAX_CHUNKS * 2
    floats.  With ``slots`` and ``feedback`` the choice is also stored in ``feedback[slots[r]]``."""
    lib = library()
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and scratch.dtype == torch.float32
    _i32(slots, "slots"); _i32(feedback, "feedback")
    assert (slots is None) == (feedback is None)
    m, v = logits.shape
    assert scratch.numel() >= m * ARGMAX_CHUNKS * 2
    _check(lib.hfee_argmax(logits.data_ptr(), _rows(logits, "logits"), m, v, ARGMAX_CHUNKS, scratch.data_ptr(),
                           out.data_ptr(), _ptr(slots), _ptr(feedback), _stream()), lib)
    count_launches(1)


# the entry points the parts and the sampler launch through can be left out by class (see tag())
for _name in ("rmsnorm_add_norm", "latent_attention", "linear_act", "attention_simt_general", "rope_norm_cache", "latent_norm_rope_cache", "head_linear", "conv_act", "delta_rule",
              "head_norm_gate", "unary_act", "head_gate", "attention_simt_masked", "short_conv", "linear_attention", "rmsnorm_add", "norm_gate", "gated_act", "scale_", "cast_rows", "sigmoid_attention",
              "qk_norm_rope_cache", "embed", "rmsnorm", "rope_table", "rope_cache_write", "swiglu", "linear", "linear_normed", "linear_swiglu", "linear_rope_cache",
              "linear_swiglu_normed", "paged_attention", "paged_attention_rope", "sample", "argmax", "sample_chain",
              "mingru", "selective_scan", "distance_attention", "moe_route", "moe_plan", "moe_experts", "moe_experts_grouped", "moe_combine",
              "clamped_glu", "linear_clamped_glu", "depth_average", "scaled_add_norm", "scaled_add", "add_sinusoid", "softcap_"):
    globals()[_name] = _measurable(globals()[_name])
del _name
