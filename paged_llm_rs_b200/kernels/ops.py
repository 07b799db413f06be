"""Python side of the CUDA kernels: argument checks, then the C entry point.

Every function takes torch tensors that live on the GPU, checks dtype, shape and
contiguity, and launches on torch's current stream.  There is no fallback: if
the kernel library cannot be built or loaded, or a tensor is not on a CUDA
device, a ``KernelError`` is raised.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import KernelError

_F32, _BF16 = 0, 1
_ERRORS = {
    -1: "dtype is neither float32 nor bfloat16",
    -2: "a size the kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "a size beyond the kernel's stated maximum",
}

_lib = None
LAUNCHES = 0  # kernels of this library launched so far (library matrix products are not counted)
c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def lib():
    global _lib
    if _lib is None:
        L = load_library()
        P = c_void_p
        sig = {
            "pllm_embed": [c_int, P, P, P, c_int, c_int, c_int, P, P],
            "pllm_rmsnorm": [c_int, P, P, P, P, P, P, c_int, c_int, c_float, P],
            "pllm_swiglu": [c_int, P, P, c_int, c_int, c_int, c_float, P],
            "pllm_qk_norm_rope_kv": [c_int, P, P, P, P, c_float, P, P, c_int, c_int, P, P, P, P,
                                     c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P],
            "pllm_attention_generic": [c_int, P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_float, P, P],
            "pllm_attention_generic_tile_tokens": [c_int, c_int],
            "pllm_attention_reduce": [c_int, P, P, P, P, c_int, P, c_int, c_int, c_int, P],
            "pllm_sample": [P, c_int, c_int, c_ll, P, P, P, P, P],
            "pllm_sample_scratch_floats": [c_int, c_int],
            "pllm_skinny_gemm_supports": [c_int, c_int, c_int],
            "pllm_skinny_gemm": [P, P, P, c_int, c_int, c_int, c_int, P],
            "pllm_skinny_gemm_act": [P, P, P, c_int, c_int, c_int, c_int, c_int, P],
            "pllm_skinny_gemm_glu_supports": [c_int, c_int, c_int],
            "pllm_skinny_gemm_glu": [P, P, P, c_int, c_int, c_int, c_int, c_float, P],
            "pllm_sm_count": [],
            "pllm_attention_mma_supports": [c_int, c_int, c_int, c_int],
            "pllm_attention_mma_tile_tokens": [c_int, c_int],
            "pllm_attention_mma": [P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_float, c_int, c_int, P, P],
            "pllm_attention_decode_tma_supports": [c_int, c_int, c_int, c_int, c_int, c_int],
            "pllm_attention_decode_tma": [P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, P, P],
        }
        sig["pllm_set_pdl"] = [c_int]
        sig["pllm_attention_decode_tma_fused"] = [P, P, P, c_float, P, P, c_int, P, P, P, P, P, c_int, P, P, P] + [c_int] * 6 + [c_float, P, P]
        sig["pllm_attention_prefill_tcgen05_tile_tokens"] = [c_int, c_int]
        sig["pllm_attention_prefill_tcgen05_supports"] = [c_int] * 6
        sig["pllm_attention_prefill_tcgen05"] = [P] * 10 + [c_int] * 7 + [c_float, c_int, P, P]
        sig["pllm_gemm_tcgen05_supports"] = [c_int, c_int, c_int, c_int]
        sig["pllm_gemm_tcgen05"] = [P, P, P, c_int, c_int, c_int, c_int, c_float, P, P]
        sig["pllm_embed_scaled32"] = [c_int, P, P, P, c_int, c_int, c_int, c_float, P, P]
        sig["pllm_sinusoid_add"] = [P, P, P, c_int, c_int, P]
        sig["pllm_round_rows"] = [c_int, P, P, c_ll, P]
        sig["pllm_outnorm_add"] = [c_int, P, P, P, P, c_int, c_int, c_float, P]
        sig["pllm_rmsnorm_from32"] = [c_int, P, P, P, P, c_int, c_int, c_float, P]
        sig["pllm_latent_norm_write"] = [c_int, P, P, P, c_float, P, P, P, c_int, c_int, c_int, c_ll, P, P]
        sig["pllm_latent_attention_generic_tile_tokens"] = [c_int]
        sig["pllm_latent_attention_generic_ctas_per_item"] = [c_int]
        sig["pllm_latent_attention_generic"] = [c_int, P, P, P, P, P, c_int, P, P, P] + [c_int] * 5 + [c_float, P, P]
        sig["pllm_latent_attention_mma_supports"] = [c_int, c_int, c_int]
        sig["pllm_latent_attention_mma_tile_tokens"] = [c_int]
        sig["pllm_latent_attention_mma_ctas_per_item"] = [c_int]
        sig["pllm_latent_attention_mma"] = [P, P, P, P, P, c_int, P, P, P] + [c_int] * 5 + [c_float, P, P]
        sig["pllm_moe_route"] = [c_int, P, P, P, P, P] + [c_int] * 6 + [P, c_int, P, c_int, P]
        sig["pllm_moe_align"] = [P, c_int, c_int, P, P, P, c_int, P]
        sig["pllm_moe_gather"] = [c_int, P, P, P, P, c_int, c_int, c_int, P, P]
        sig["pllm_moe_combine"] = [c_int, P, P, P, P, P, P, c_int, c_int, c_int, P, c_int, P]
        sig["pllm_gemm_tcgen05_grouped"] = [P, P, P, c_int, c_int, c_int, c_int, c_float, P, c_int, P, P]
        sig["pllm_moe_pair_glu"] = [c_int, P, P, P, P] + [c_int] * 6 + [c_float, c_int, P, P]
        sig["pllm_moe_pair_down"] = [c_int, P, P, P, P, P, P, P] + [c_int] * 5 + [P, c_int, P]
        sig["pllm_embed_norm32"] = [c_int, P, P, P, P, c_int, c_int, c_int, c_float, P, P]
        sig["pllm_add_scaled_norm32"] = [c_int, P, P, c_float, P, P, P, c_int, c_int, c_float, P]
        sig["pllm_add_scaled32"] = [c_int, P, P, c_float, c_ll, P]
        sig["pllm_scale32"] = [P, c_float, c_ll, P]
        sig["pllm_rope_mix_kv_write"] = [c_int, P, c_int, P, P, c_int, P, P, P, P, c_int, P] + [c_int] * 6 + [c_ll, P, P]
        sig["pllm_attention_sink"] = [c_int, P, P, P, P, P, c_int, P, P, P, P] + [c_int] * 9 + [c_float, c_float, P, P]
        sig["pllm_attention_sink_tile_tokens"] = [c_int, c_int]
        sig["pllm_attention_sink_mma_supports"] = [c_int] * 5
        sig["pllm_attention_sink_mma_tile_tokens"] = [c_int, c_int]
        sig["pllm_attention_sink_mma"] = [P, P, P, P, P, c_int, P, P, P, P] + [c_int] * 9 + [c_float, c_float, P, P]
        sig["pllm_mamba2_mix"] = [c_int] + [P] * 8 + [c_int, c_int, P, c_ll, P, P, P] + [c_int] * 7 + [c_float, P]
        sig["pllm_pack_decode_step"] = [P, c_int, c_int, P, P, P, P, P] + [c_int] * 16 + [P, P]
        sig["pllm_sandwich_norm32"] = [c_int, P, P, P, P, P, P, P, c_int, c_int, c_float, P]
        sig["pllm_scaled_sum2"] = [c_int, P, P, c_float, c_float, P, c_ll, P]
        sig["pllm_swiglu_bias"] = [c_int, P, P, P, c_int, c_int, c_int, c_float, P]
        sig["pllm_normed_qk_kv_write"] = [c_int, P, c_int, c_int, c_int, P, P, P, c_int, c_float, c_float, c_int, P, c_int, P, P, P] + [c_int] * 7 + [c_ll, P, P]
        sig["pllm_gate_mul"] = [c_int, P, P, c_int, c_int, c_int, c_int, c_int, P]
        sig["pllm_unary_act"] = [c_int, P, c_ll, c_int, P]
        sig["pllm_conv_rope_kv_write"] = [c_int, P, c_int, P, P, c_int, P, c_int, c_int, P, c_ll, P, c_int, P, P, P, P] + [c_int] * 6 + [c_ll, P, P]
        sig["pllm_diff_combine"] = [c_int, P, P, c_int, P] + [c_int] * 4 + [c_float] * 3 + [P]
        sig["pllm_latent_rope_write"] = [c_int, P, c_int, P, c_float, P, c_int, P, P, P, P, P, P, P] + [c_int] * 6 + [c_ll, P, P]
        sig["pllm_mlstm_mix"] = [c_int, P, c_int, P, P, P, c_float, P, P, c_int, c_int, P, c_ll, P, P, P, P] + [c_int] * 4 + [c_float, P]
        sig["pllm_delta_mix"] = [c_int, P, c_int, P, P, P, P, P, P, c_int, c_int, P, c_ll, P, P, P] + [c_int] * 6 + [c_float, P]
        wide = {"pllm_mlstm_state_floats": [c_int] * 3, "pllm_delta_state_floats": [c_int] * 5}
        for name, args in wide.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_ll
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        # The kernels are launched with programmatic dependent launch: a kernel's CTAs
        # may take their places while the one before it drains (the long kernels let
        # them in after their main loops; every kernel waits for its predecessors
        # before it touches memory).  A decode step measured 11% faster with it;
        # PAGED_LLM_PDL=0 turns it off.
        L.pllm_set_pdl(0 if os.environ.get("PAGED_LLM_PDL", "1") == "0" else 1)
        _lib = L
    return _lib


def _check(code: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += launches
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {t.dtype} is not handled: the kernels take float32 and bfloat16")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("a tensor is not on a CUDA device: there is no CPU path")
        if not t.is_contiguous():
            raise KernelError("a tensor is not contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


def _f32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{name} must be float32, got {t.dtype}")


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]]; tokens int32 [T], table [V, H], out [T, H]."""
    _dev(tokens, table, out, status)
    _i32(tokens, "tokens")
    T, (V, H) = tokens.numel(), table.shape
    if out.shape != (T, H) or out.dtype != table.dtype:
        raise KernelError(f"embed: out is {tuple(out.shape)} {out.dtype}, expected {(T, H)} {table.dtype}")
    _check(lib().pllm_embed(_code(table), _ptr(tokens), _ptr(table), _ptr(out), T, H, V, _ptr(status), _stream()),
           "embed")
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rmsnorm(x[r] (+ delta[r])) * gain with r = rows[i] or i; when
    residual_out is given the sum is stored to residual_out[r] (may alias x)."""
    _dev(x, gain, out, delta, residual_out, rows)
    _f32(gain, "gain")
    _i32(rows, "rows")
    W = x.shape[-1]
    n = rows.numel() if rows is not None else x.numel() // W
    if gain.numel() != W:
        raise KernelError(f"rmsnorm: gain has {gain.numel()} entries for rows of width {W}")
    if out.numel() != n * W or out.dtype != x.dtype:
        raise KernelError("rmsnorm: out does not fit")
    for t in (delta, residual_out):
        if t is not None and (t.shape != x.shape or t.dtype != x.dtype):
            raise KernelError("rmsnorm: delta / residual_out must have x's shape and dtype")
    _check(lib().pllm_rmsnorm(_code(x), _ptr(x), _ptr(delta), _ptr(residual_out), _ptr(gain), _ptr(out),
                              _ptr(rows), n, W, float(eps), _stream()), "rmsnorm")
    return out


# The gated activations y = act(g, u) (csrc/common.cuh): silu(g) u; max(g, 0) u; and, with g' = min(g, limit) and
# u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1).
GLU_KINDS = {"silu": 0, "relu": 1, "clamped": 2}


def _glu(act: str) -> int:
    try:
        return GLU_KINDS[act]
    except KeyError:
        raise KernelError(f"gated activation {act!r} is not known; known: {sorted(GLU_KINDS)}") from None


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """out[n, I] = act(gate_up[n, :I], gate_up[n, I:]), silu(g) * u unless ``act`` names another gated activation."""
    _dev(gate_up, out)
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: out must be [n, I] for an input [n, 2I] of the same dtype")
    _check(lib().pllm_swiglu(_code(gate_up), _ptr(gate_up), _ptr(out), n, two_i // 2, _glu(act), float(limit), _stream()), "swiglu")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, q_gain, k_gain, eps: float, cos, sin,
                    rotary_dim: int, positions: torch.Tensor, slots: torch.Tensor, k_pool, v_pool,
                    num_heads: int, num_kv_heads: int, head_dim: int, status: torch.Tensor,
                    swizzled: bool = False) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation, q to q_out, k and v into the paged
    pools [pages, kv_heads, page_size, head_dim] at ``slots`` (a negative slot, or
    k_pool None, writes nothing).  ``swizzled``: the pools keep each row's 16-byte
    chunks at chunk ^ (offset in page & 7), the layout of ``pool_is_swizzled``."""
    _dev(qkv, q_out, q_gain, k_gain, cos, sin, positions, slots, k_pool, v_pool, status)
    _f32(q_gain, "q_gain"); _f32(k_gain, "k_gain"); _f32(cos, "cos"); _f32(sin, "sin")
    _i32(positions, "positions"); _i32(slots, "slots")
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (T, width):
        raise KernelError(f"qk_norm_rope_kv: qkv is {tuple(qkv.shape)}, expected {(T, width)}")
    if q_out.numel() != T * num_heads * head_dim or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_kv: q_out does not fit")
    if positions.numel() < T or slots.numel() < T:
        raise KernelError("qk_norm_rope_kv: positions / slots shorter than the tokens")
    max_pos, page_size, n_pages = 0, 1, 0
    if cos is not None:
        if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_kv: cos/sin must be [max_positions, rotary_dim/2]")
        max_pos = cos.shape[0]
    if k_pool is not None:
        if k_pool.shape != v_pool.shape or k_pool.dtype != qkv.dtype or k_pool.dim() != 4 \
                or k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim:
            raise KernelError(f"qk_norm_rope_kv: pools must be [pages, {num_kv_heads}, page_size, {head_dim}] "
                              f"of {qkv.dtype}, got {tuple(k_pool.shape)} {k_pool.dtype}")
        n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    for g in (q_gain, k_gain):
        if g is not None and g.numel() != head_dim:
            raise KernelError("qk_norm_rope_kv: a head gain must have head_dim entries")
    _check(lib().pllm_qk_norm_rope_kv(_code(qkv), _ptr(qkv), _ptr(q_out), _ptr(q_gain), _ptr(k_gain), float(eps),
                                      _ptr(cos), _ptr(sin), rotary_dim, max_pos, _ptr(positions), _ptr(slots),
                                      _ptr(k_pool), _ptr(v_pool), T, num_heads, num_kv_heads, head_dim, page_size,
                                      n_pages, 1 if swizzled else 0, _ptr(status), _stream()), "qk_norm_rope_kv")
    return q_out


def attention_uses_tensor_cores(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether paged_attention runs the mma kernel for this shape (bfloat16, head
    sizes 64 and 128) or the generic one."""
    if dtype != torch.bfloat16:
        return False
    return bool(lib().pllm_attention_mma_supports(_BF16, num_heads, num_kv_heads, head_dim))


TMA_KINDS = int(os.environ.get("PAGED_LLM_TMA_KINDS", "3"))  # which items the bulk-copy attention kernel takes where it applies: 1 single tokens, 2 portions, 3 both


def pool_is_swizzled(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the cache pools of such layers keep each row's 16-byte chunks at
    chunk ^ (offset in page & 7).  True exactly where the tensor-core attention
    kernels run: they read that layout from shared memory without bank conflicts,
    and the decode kernel copies whole pages there as they lie."""
    return attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim)


def swizzle_pool_(pool: torch.Tensor) -> torch.Tensor:
    """Rearrange a plain pool [pages, kv_heads, page_size, head_dim] into the swizzled
    layout in place (its own inverse); for tests and tools."""
    pages, nkv, ps, hd = pool.shape
    epc = 16 // pool.element_size()
    ch = hd // epc
    if ch % 8:
        raise KernelError("swizzle_pool_: a row must hold a multiple of eight 16-byte chunks")
    v = pool.view(pages, nkv, ps, ch, epc)
    o = torch.arange(ps, device=pool.device)[:, None] & 7
    c = torch.arange(ch, device=pool.device)[None, :]
    idx = (c ^ o)[None, None, :, :, None].expand_as(v)
    pool.copy_(torch.gather(v.clone(), 3, idx).view_as(pool))
    return pool


# Prompt portions (work items of several tokens) in bfloat16 over swizzled pages: the tcgen05 kernel
# (csrc/attention_prefill_tcgen05.cu), 128 rows an item (PAGED_LLM_TCGEN05_ATTN=0: the mma.sync kernels).
TCGEN05_ATTN = os.environ.get("PAGED_LLM_TCGEN05_ATTN", "1") != "0"


def attention_prefill_uses_tcgen05(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: Optional[int],
                                   window: int) -> bool:
    if not TCGEN05_ATTN or page_size is None or not pool_is_swizzled(dtype, num_heads, num_kv_heads, head_dim):
        return False
    return bool(lib().pllm_attention_prefill_tcgen05_supports(_BF16, num_heads, num_kv_heads, head_dim, int(page_size),
                                                              int(window or 0)))


def attention_tile_tokens(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32,
                          head_dim: int = 0, page_size: Optional[int] = None, window: int = 0) -> int:
    """The most query tokens one attention work item may hold, for the kernel that
    paged_attention picks for this dtype, shape and (when given) cache layout."""
    if attention_prefill_uses_tcgen05(dtype, num_heads, num_kv_heads, head_dim, page_size, window):
        return lib().pllm_attention_prefill_tcgen05_tile_tokens(num_heads, num_kv_heads)
    if attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim):
        return lib().pllm_attention_mma_tile_tokens(num_heads, num_kv_heads)
    return lib().pllm_attention_generic_tile_tokens(num_heads, num_kv_heads)


# PAGED_LLM_MIXED_BESIDE=0: in a step of decoded tokens beside prompt portions the tcgen05 kernel takes the
# single tokens too (one launch) instead of the bulk-copy kernel running beside it on a second stream.
MIXED_BESIDE = os.environ.get("PAGED_LLM_MIXED_BESIDE", "1") != "0"
MIXED_BESIDE_MIN_REQUESTS = 9       # rows of the step's block tables (a captured step's capacity)
MIXED_BESIDE_CALLS = 0              # how often that route was taken (for tests)
_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index or 0
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


def sm_count() -> int:
    """Streaming multiprocessors of the current device (the kernels size their grids by it)."""
    return int(lib().pllm_sm_count())


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor, w,
                    out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                    status: torch.Tensor, swizzled: bool = False) -> torch.Tensor:
    """Attention of the step's tokens over the paged cache, then the reduction of
    split items.  ``w`` is the group's ``AttentionWork`` (parts/base.py): work items
    int32 [>=max_work, 8], reductions int32 [>=max_red, 4], how many are live as
    int32 scalars on the device, the scratch for partial results, and ``kinds``,
    what the work items are (1 single decoded tokens only, 2 portions of several
    tokens only, 3 both), so that only the kernels with work are launched.
    ``swizzled`` says how the pools are laid out (see ``pool_is_swizzled``)."""
    work, n_work, max_work, red, n_red, max_red = w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red
    part_o, part_ml, kinds = w.part_o, w.part_ml, w.kinds
    _dev(q, k_pool, v_pool, block_tables, work, n_work, out, part_o, part_ml, red, n_red, status)
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml")
    if k_pool.dtype != q.dtype or out.dtype != q.dtype or k_pool.shape != v_pool.shape:
        raise KernelError("paged_attention: q, pools and out must share one dtype, pools one shape")
    if k_pool.dim() != 4 or k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim:
        raise KernelError(f"paged_attention: pools must be [pages, {num_kv_heads}, page_size, {head_dim}]")
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"paged_attention: head_dim {head_dim} is not a multiple of 16 up to 256")
    if num_heads % num_kv_heads:
        raise KernelError(f"paged_attention: {num_heads} heads do not group over {num_kv_heads} kv heads")
    if work.numel() < max_work * 8 or red.numel() < max_red * 4:
        raise KernelError("paged_attention: work / red lists shorter than their maxima")
    if part_o.shape[1:] != (num_heads, head_dim) or part_ml.shape[1:] != (num_heads, 2):
        raise KernelError("paged_attention: the scratch for partial results is not [rows, heads, head_dim] and [rows, heads, 2]")
    n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    L = lib()
    if attention_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim):
        # The bulk-copy kernel where the cache layout allows it (swizzled rows, pages of a power
        # of two tokens, no window); TMA_KINDS says which items it takes there: 1 single decoded
        # tokens, 2 portions of several tokens, 3 both.  The cp.async kernel takes the rest.
        tma_ok = swizzled and bool(L.pllm_attention_decode_tma_supports(_BF16, num_heads, num_kv_heads, head_dim,
                                                                        page_size, int(window)))
        # portions of several tokens go to the tcgen05 kernel where the layout allows it
        multi_tc = bool(kinds & 2) and swizzled and attention_prefill_uses_tcgen05(q.dtype, num_heads, num_kv_heads, head_dim,
                                                                                   page_size, int(window))
        # (worth the two edges without programmatic launch from some eight requests on: 0.6B shape, a layer of a
        # step of 1 / 8 / 64 decoded tokens at 4096 beside a portion: +9 / -3 / -10 us)
        beside = bool(MIXED_BESIDE and multi_tc and kinds == 3 and tma_ok and (TMA_KINDS & 1)
                      and block_tables.shape[0] >= MIXED_BESIDE_MIN_REQUESTS)
        if beside:
            # A step of decoded tokens beside prompt portions: the single tokens go to the bulk-copy kernel and
            # the portions to the tcgen05 kernel, on two streams that meet again before the reduction.  Neither
            # kernel reads what the other writes, a CTA of one does not fit an SM beside a CTA of the other, and
            # the single tokens' long key ranges no longer queue behind tiles of 128 rows with two of them live.
            global MIXED_BESIDE_CALLS
            MIXED_BESIDE_CALLS += 1
            main, side = torch.cuda.current_stream(), _side_stream(q.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                _check(L.pllm_attention_decode_tma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                                   _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                                   num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                                   block_tables.shape[-1], float(scale), 1, _ptr(status), _stream()),
                       "paged_attention (bulk copy, beside)")
        if multi_tc:
            _check(L.pllm_attention_prefill_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                                    _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                                    q.shape[0], num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                                    block_tables.shape[-1], float(scale), 1 if (kinds == 3 and not beside) else 0,
                                                    _ptr(status), _stream()),
                   "paged_attention (tcgen05)")
            if beside:
                torch.cuda.current_stream().wait_stream(_side_stream(q.device))
            # (else) beside portions it takes the single decoded tokens too: one launch a layer, not two
            kinds = 0 if kinds == 3 else kinds & ~2
        take = (kinds & TMA_KINDS) if tma_ok else 0
        rest = kinds & ~take
        if take:
            _check(L.pllm_attention_decode_tma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                               _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                               num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                               block_tables.shape[-1], float(scale), take, _ptr(status), _stream()),
                   "paged_attention (bulk copy)")
        if rest:
            _check(L.pllm_attention_mma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                        _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml), num_heads,
                                        num_kv_heads, head_dim, page_size, n_pages, block_tables.shape[-1], int(window),
                                        float(scale), 1 if swizzled else 0, rest, _ptr(status), _stream()),
                   "paged_attention (mma)")
    else:
        if swizzled:
            raise KernelError("paged_attention: the generic kernel reads plain pools, not swizzled ones")
        _check(L.pllm_attention_generic(_code(q), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables),
                                        _ptr(work), _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                        num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                        block_tables.shape[-1], int(window), float(scale), _ptr(status), _stream()),
               "paged_attention")
    _check(L.pllm_attention_reduce(_code(q), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red,
                                   _ptr(out), num_heads, head_dim, 1 if w.many_splits else 0, _stream()), "attention_reduce")
    return out


# A step of single decoded tokens: the q/k norm, the rotation and the cache write are done by the
# attention kernel itself (PAGED_LLM_FUSE_QK=0: by their own kernel before it, as for prompt portions).
FUSE_QK = os.environ.get("PAGED_LLM_FUSE_QK", "1") != "0"


def decode_attention_fuses(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                           rotary_dim: int, swizzled: bool) -> bool:
    """Whether ``decode_attention_fused`` takes a step of single tokens of this shape: the bulk-copy
    kernel's conditions, and a rotation over the whole head or none."""
    if not FUSE_QK or not swizzled or not (TMA_KINDS & 1) or rotary_dim not in (0, head_dim):
        return False
    if not attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim):
        return False
    return bool(lib().pllm_attention_decode_tma_supports(_BF16, num_heads, num_kv_heads, head_dim, int(page_size),
                                                         int(window or 0)))


def decode_attention_fused(qkv: torch.Tensor, q_gain, k_gain, eps: float, cos, sin, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, block_tables: torch.Tensor, w, out: torch.Tensor, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float, status: torch.Tensor) -> torch.Tensor:
    """Attention of a step of single decoded tokens straight from the projection's output
    ``qkv`` [tokens, (heads + 2 kv heads) * head_dim]: per-head norm of q and k, rotation at each
    token's position (the work item's), the token's key and value written to its cache slot
    (found through the block table), attention over the cache, reduction of split items.
    ``w``: the group's ``AttentionWork``."""
    work, n_work, max_work, red, n_red, max_red, part_o, part_ml = (w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red,
                                                                    w.part_o, w.part_ml)
    _dev(qkv, k_pool, v_pool, block_tables, work, n_work, out, part_o, part_ml, red, n_red, status, q_gain, k_gain, cos, sin)
    _f32(q_gain, "q_gain"); _f32(k_gain, "k_gain"); _f32(cos, "cos"); _f32(sin, "sin")
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml")
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    if qkv.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention_fused: bfloat16 only")
    if qkv.shape[-1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("decode_attention_fused: qkv's width is not (heads + 2 kv heads) * head_dim")
    if (cos is None) != (sin is None) or (cos is not None and cos.shape[-1] * 2 != head_dim):
        raise KernelError("decode_attention_fused: the rotation must span the whole head (or be absent)")
    n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    L = lib()
    _check(L.pllm_attention_decode_tma_fused(_ptr(qkv), _ptr(q_gain), _ptr(k_gain), float(eps), _ptr(cos), _ptr(sin),
                                             cos.shape[0] if cos is not None else 0, _ptr(k_pool), _ptr(v_pool),
                                             _ptr(block_tables), _ptr(work), _ptr(n_work), max_work, _ptr(out),
                                             _ptr(part_o), _ptr(part_ml), num_heads, num_kv_heads, head_dim, page_size,
                                             n_pages, block_tables.shape[-1], float(scale), _ptr(status), _stream()),
           "decode_attention_fused")
    _check(L.pllm_attention_reduce(_code(out), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red,
                                   _ptr(out), num_heads, head_dim, 1 if w.many_splits else 0, _stream()), "attention_reduce")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """tokens[i] = argmax(logits[i]) where temperature[i] <= 0, else a draw from
    softmax(logits[i] / temperature[i]) at uniform[i], walking ids upward."""
    _dev(logits, temperature, uniform, tokens)
    _f32(logits, "logits"); _f32(temperature, "temperature"); _f32(uniform, "uniform"); _i32(tokens, "tokens")
    n, V = logits.shape
    if min(temperature.numel(), uniform.numel(), tokens.numel()) < n:
        raise KernelError("sample: per-row arguments shorter than the rows")
    L = lib()
    # per chunk of a row (max, first index of it, sum): scratch between the two launches
    scratch = torch.empty(L.pllm_sample_scratch_floats(n, V), dtype=torch.float32, device=logits.device)
    _check(L.pllm_sample(_ptr(logits), n, V, logits.stride(0), _ptr(temperature), _ptr(uniform), _ptr(tokens),
                         _ptr(scratch), _stream()), "sample", launches=2)
    return tokens


SKINNY_GEMM = True  # few rows in bfloat16 go to this library's weight-streaming kernel
FUSE_GLU = os.environ.get("PAGED_LLM_FUSE_GLU", "1") != "0"     # ... with the gated activation in its epilogue


def skinny_gemm_takes(x: torch.Tensor, weight: torch.Tensor, k: Optional[int] = None) -> bool:
    """Whether ``linear`` runs the weight-streaming kernel for this product."""
    if not SKINNY_GEMM or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    N, K = weight.shape
    return x.shape[0] <= SKINNY_MAX_M and bool(lib().pllm_skinny_gemm_supports(x.shape[0], N, K if k is None else k))


# Measured on a B200 inside a captured step (0.6B shapes, microseconds, skinny / cuBLAS):
#   rows 1-8:  qkv 3.5-3.8 / 5.0   o 3.1 / 6.4-7.5   gate_up 4.6-4.8 / 5.1   down 3.9-4.2 / 8.9-9.6
#   rows 64:   qkv 12.3 / 4.9      o 6.3 / 5.4        gate_up 12.6 / 5.3      down 8.4 / 6.6
# so the kernel (which takes up to 64 rows) is used up to 16, and up to a width where the
# library's head product is the faster one (151936 x 1024: 66 / 54).
SKINNY_MAX_M = 16
SKINNY_MAX_N = 32768


# The many rows of a prompt portion in bfloat16: this library's tcgen05 product (csrc/gemm_tcgen05.cu)
# where it is the faster one.  Measured on a B200 at 2048 rows (us, this kernel / cuBLAS):
#   gate/up 6144 x 1024 with silu(gate)*up in the epilogue 25.2 / 24.3 + 10.8 for the activation's own pass
#   qkv 4096 x 1024   18.5 / 17.7      o 1024 x 2048   17.4 / 10.7      down 1024 x 3072   19.5 / 12.6
# so the gated product takes it and the plain ones stay with the library (PAGED_LLM_TCGEN05=0: none,
# =2: the plain ones too).  One CTA's tcgen05.mma reads both operands from shared memory, whose
# bandwidth bounds a 128 x 256 tile at two thirds of the tensor peak; pairs of CTAs are the next step.
TCGEN05_GEMM = int(os.environ.get("PAGED_LLM_TCGEN05", "1"))
TCGEN05_MIN_M = 64     # below this the tiles of 128 rows are mostly padding
_gemm_status: dict = {}


def gemm_status(device) -> torch.Tensor:
    """The status word the tcgen05 product raises bit 64 in when one of its bounded waits
    ran out (one int32 per device; the engine reads it with its own status word)."""
    key = str(device)
    if key not in _gemm_status:
        _gemm_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _gemm_status[key]


def gemm_tcgen05_takes(x, weight: torch.Tensor, n_out: int, glu: bool) -> bool:
    if not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    return x.is_contiguous() and weight.is_contiguous() and bool(
        lib().pllm_gemm_tcgen05_supports(x.shape[0], n_out, weight.shape[1], 1 if glu else 0))


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, glu: bool = False, status: Optional[torch.Tensor] = None,
                 act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """x W^T on the tcgen05 tensor cores (bfloat16, float accumulation); with ``glu`` W is
    [gate rows; up rows] and the result is silu(x Wg^T) * (x Wu^T)."""
    M, K = x.shape
    n_out = weight.shape[0] // 2 if glu else weight.shape[0]
    if weight.shape[1] != K or not gemm_tcgen05_takes(x, weight, n_out, glu):
        raise KernelError(f"gemm_tcgen05: does not take x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)} {weight.dtype}")
    _dev(x, weight)
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    st = status if status is not None else gemm_status(x.device)
    _check(lib().pllm_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), M, n_out, K, 1 + _glu(act) if glu else 0, float(limit),
                                   _ptr(st), _stream()), "gemm_tcgen05")
    return out


def skinny_glu_takes(x, weight: torch.Tensor, n_out: int) -> bool:
    """Whether the weight-streaming kernel takes the gate/up product with the activation in its epilogue."""
    if not SKINNY_GEMM or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    return n_out <= SKINNY_MAX_N and bool(lib().pllm_skinny_gemm_glu_supports(x.shape[0], n_out, weight.shape[1]))


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, gated: bool = False,
           out_dtype: Optional[torch.dtype] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T with W stored [out, in].

    Few rows (a decode step) in bfloat16 run this library's weight-streaming
    kernel.  With ``gated`` the input is [g | u] of twice W's width and the
    product is taken of silu(g) * u, formed by the activation kernel first.
    Everything else is the library matrix product (cuBLAS through torch), which
    is where the reference uses a library too
    (crates/pagedllm/src/model/layers.rs:27-35).  float32 inputs run in true
    float32: the engine switches TF32 off."""
    N, K = weight.shape
    if not x.is_cuda:
        raise KernelError("linear: input is not on a CUDA device: there is no CPU path")
    if x.shape[-1] != (2 * K if gated else K):
        raise KernelError(f"linear: input width {x.shape[-1]} does not fit a weight of {tuple(weight.shape)}")
    want = out_dtype or x.dtype
    if gated:
        # Forming silu(g) * u inside the product that consumes it repeats it in every CTA
        # (measured 31 us against 3.4 + 6 us at batch 8, 3072 -> 1024): a pass of its own here,
        # or the epilogue of the product that makes [g | u] (linear_glu).
        act = torch.empty((x.shape[0], K), dtype=x.dtype, device=x.device)
        swiglu(x, act)
        x = act
    # The widest products (the output head) stay with the library, which is faster there
    # (measured 54 us against 66 us at 151936 x 1024, batch 8).
    if skinny_gemm_takes(x, weight, K) and N <= SKINNY_MAX_N and want in (torch.bfloat16, torch.float32):
        _dev(x, weight, out)
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        elif out.shape != (M, N) or out.dtype != want:
            raise KernelError("linear: out does not fit")
        _check(lib().pllm_skinny_gemm(_ptr(x), _ptr(weight), _ptr(out), M, N, K,
                                      1 if want == torch.float32 else 0, _stream()), "skinny_gemm")
        return out
    if TCGEN05_GEMM >= 2 and out is None and want == torch.bfloat16 and x.shape[0] >= TCGEN05_MIN_M \
            and gemm_tcgen05_takes(x, weight, N, False):
        return gemm_tcgen05(x, weight, status=status)
    if want != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=want)
    return torch.matmul(x, weight.t(), out=out) if out is not None else torch.matmul(x, weight.t())


def linear_glu(x: torch.Tensor, w_gate_up: torch.Tensor, status: Optional[torch.Tensor] = None, act: str = "silu",
               limit: float = 0.0) -> torch.Tensor:
    """act(x Wg^T, x Wu^T), silu(g) * u unless ``act`` says otherwise, for W = [Wg; Wu] stacked [2I, K]: the gated
    feed-forward's first half (crates/pagedllm/src/model/layers.rs:93-99).  Few
    rows in bfloat16: one kernel whose CTAs hold the same columns of both halves;
    many rows: the tcgen05 product with the activation in its epilogue; otherwise
    the product, then the activation kernel."""
    two_i, K = w_gate_up.shape
    if two_i % 2:
        raise KernelError("linear_glu: the stacked weight needs an even number of rows")
    inter = two_i // 2
    if x.shape[-1] != K:
        raise KernelError(f"linear_glu: input width {x.shape[-1]} does not fit a weight of {tuple(w_gate_up.shape)}")
    if FUSE_GLU and skinny_glu_takes(x, w_gate_up, inter):
        _dev(x, w_gate_up)
        out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
        _check(lib().pllm_skinny_gemm_glu(_ptr(x), _ptr(w_gate_up), _ptr(out), x.shape[0], inter, K, _glu(act), float(limit),
                                          _stream()), "skinny_gemm_glu")
        return out
    if TCGEN05_GEMM >= 1 and x.shape[0] >= TCGEN05_MIN_M and gemm_tcgen05_takes(x, w_gate_up, inter, True):
        return gemm_tcgen05(x, w_gate_up, glu=True, status=status, act=act, limit=limit)
    gu = linear(x, w_gate_up)
    return swiglu(gu, torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device), act, limit)


# ---- a residual stream kept in float32 (csrc/stream32.cu) ---------------------------------------------

def _code_of(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {dtype} is not handled: the kernels take float32 and bfloat16")


def embed_scaled32(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale as float32, whatever the table's dtype."""
    _dev(tokens, table, out, status)
    _i32(tokens, "tokens"); _f32(out, "out")
    T, (V, H) = tokens.numel(), table.shape
    if out.shape != (T, H):
        raise KernelError(f"embed_scaled32: out is {tuple(out.shape)}, expected {(T, H)}")
    _check(lib().pllm_embed_scaled32(_code(table), _ptr(tokens), _ptr(table), _ptr(out), T, H, V, float(scale), _ptr(status),
                                     _stream()), "embed_scaled32")
    return out


def sinusoid_add(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x[t, 2i] += sin(p_t f_i), x[t, 2i + 1] += cos(p_t f_i) in place; x float32 [T, width], inv_freq float32 [width / 2]."""
    _dev(x, positions, inv_freq)
    _f32(x, "x"); _f32(inv_freq, "inv_freq"); _i32(positions, "positions")
    T, W = x.shape
    if inv_freq.numel() * 2 != W or positions.numel() < T:
        raise KernelError("sinusoid_add: inv_freq must hold width / 2 entries and positions one per row")
    _check(lib().pllm_sinusoid_add(_ptr(x), _ptr(positions), _ptr(inv_freq), T, W, _stream()), "sinusoid_add")
    return x


def round_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A copy of the float32 tensor x rounded to ``dtype``."""
    _dev(x)
    _f32(x, "x")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(lib().pllm_round_rows(_code_of(dtype), _ptr(x), _ptr(out), x.numel(), _stream()), "round_rows")
    return out


def outnorm_add(x: torch.Tensor, a: torch.Tensor, gain: torch.Tensor, eps: float, h: Optional[torch.Tensor]) -> torch.Tensor:
    """x += a / sqrt(mean(a^2) + eps) * gain, row by row, x float32 in place; h (a's dtype, or None) receives x rounded."""
    _dev(x, a, gain, h)
    _f32(x, "x"); _f32(gain, "gain")
    n, W = x.shape
    if a.shape != x.shape or gain.numel() != W or (h is not None and (h.shape != x.shape or h.dtype != a.dtype)):
        raise KernelError("outnorm_add: a and h must have x's shape, gain its width")
    _check(lib().pllm_outnorm_add(_code(a), _ptr(x), _ptr(a), _ptr(gain), _ptr(h), n, W, float(eps), _stream()), "outnorm_add")
    return x


def rmsnorm_from32(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rmsnorm(x[r]) * gain for float32 x, r = rows[i] or i; out in float32 or bfloat16."""
    _dev(x, gain, out, rows)
    _f32(x, "x"); _f32(gain, "gain"); _i32(rows, "rows")
    W = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if gain.numel() != W or out.shape != (n, W):
        raise KernelError("rmsnorm_from32: out or gain does not fit")
    _check(lib().pllm_rmsnorm_from32(_code(out), _ptr(x), _ptr(gain), _ptr(out), _ptr(rows), n, W, float(eps), _stream()),
           "rmsnorm_from32")
    return out


# ---- latent attention (csrc/latent.cu) --------------------------------------------------------------------

def latent_norm_write(qa: torch.Tensor, q_gain: torch.Tensor, kv_gain: torch.Tensor, eps: float, cq: torch.Tensor,
                      pool: Optional[torch.Tensor], slots: Optional[torch.Tensor], q_rank: int, kv_rank: int,
                      status: torch.Tensor) -> torch.Tensor:
    """qa [T, q_rank + kv_rank]: RMS norm of both parts; the first to cq [T, q_rank], the second to row ``slots[t]`` of
    the paged pool [pages, page_size, kv_rank] (a negative slot, or pool None, writes nothing)."""
    _dev(qa, q_gain, kv_gain, cq, pool, slots, status)
    _f32(q_gain, "q_gain"); _f32(kv_gain, "kv_gain"); _i32(slots, "slots")
    T = qa.shape[0]
    if qa.shape != (T, q_rank + kv_rank) or cq.shape != (T, q_rank) or cq.dtype != qa.dtype:
        raise KernelError("latent_norm_write: qa must be [T, q_rank + kv_rank] and cq [T, q_rank] of one dtype")
    if q_gain.numel() != q_rank or kv_gain.numel() != kv_rank:
        raise KernelError("latent_norm_write: a gain does not fit its latent")
    rows = 0
    if pool is not None:
        if pool.dtype != qa.dtype or pool.shape[-1] != kv_rank or slots is None or slots.numel() < T:
            raise KernelError("latent_norm_write: the pool must hold rows of kv_rank values of qa's dtype, with a slot a token")
        rows = pool.numel() // kv_rank
    _check(lib().pllm_latent_norm_write(_code(qa), _ptr(qa), _ptr(q_gain), _ptr(kv_gain), float(eps), _ptr(cq), _ptr(pool),
                                        _ptr(slots), T, q_rank, kv_rank, rows, _ptr(status), _stream()), "latent_norm_write")
    return cq


# PAGED_LLM_LATENT_MMA=0: the CUDA-core kernel everywhere (for comparisons)
LATENT_MMA = os.environ.get("PAGED_LLM_LATENT_MMA", "1") != "0"


def latent_attention_uses_tensor_cores(heads: int, kv_rank: int, dtype: torch.dtype) -> bool:
    """bfloat16 with a latent of 64, 128 or 256 values: the mma.sync kernel of the grouped-query attention, with the
    one pool read as keys and as values; everything else runs the CUDA-core kernel."""
    return LATENT_MMA and dtype == torch.bfloat16 and bool(lib().pllm_latent_attention_mma_supports(_BF16, int(heads), int(kv_rank)))


def latent_attention_tile_tokens(heads: int, kv_rank: int, dtype: torch.dtype) -> int:
    """The most query tokens one work item of ``latent_attention`` may hold, for the kernel it picks."""
    if latent_attention_uses_tensor_cores(heads, kv_rank, dtype):
        return int(lib().pllm_latent_attention_mma_tile_tokens(int(heads)))
    return int(lib().pllm_latent_attention_generic_tile_tokens(int(heads)))


# How heavily a CTA of the tensor-core kernel counts when the step's attention is cut into splits: its CTAs hold
# half an SM each and pay a fixed start and a combine through shared memory, so fewer, longer splits suit it.
LATENT_CTA_WEIGHT = int(os.environ.get("PAGED_LLM_LATENT_CTA_WEIGHT", "1"))


def latent_attention_ctas_per_item(heads: int, kv_rank: int, dtype: torch.dtype) -> int:
    if latent_attention_uses_tensor_cores(heads, kv_rank, dtype):
        return int(lib().pllm_latent_attention_mma_ctas_per_item(int(heads))) * LATENT_CTA_WEIGHT
    return int(lib().pllm_latent_attention_generic_ctas_per_item(int(heads)))


def latent_attention(q: torch.Tensor, rows: torch.Tensor, block_tables: torch.Tensor, w, out: torch.Tensor, scale: float,
                     status: torch.Tensor) -> torch.Tensor:
    """Attention of every head over one shared row a cached token, the rows being keys and values at once:
    q, out [tokens, heads, R]; rows the paged pool [pages, page_size, R]; ``w`` the group's ``AttentionWork``.
    Then the reduction of split items."""
    work, n_work, max_work, red, n_red, max_red = w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red
    part_o, part_ml = w.part_o, w.part_ml
    _dev(q, rows, block_tables, work, n_work, out, part_o, part_ml, red, n_red, status)
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml")
    T, H, R = q.shape
    if rows.dim() != 3 or rows.shape[2] != R or rows.dtype != q.dtype or out.shape != q.shape or out.dtype != q.dtype:
        raise KernelError("latent_attention: q and out must be [tokens, heads, R], the pool [pages, page_size, R], of one dtype")
    if part_o.shape[1:] != (H, R) or part_ml.shape[1:] != (H, 2):
        raise KernelError("latent_attention: the scratch for partial results is not [rows, heads, R] and [rows, heads, 2]")
    if work.numel() < max_work * 8 or red.numel() < max_red * 4:
        raise KernelError("latent_attention: work / red lists shorter than their maxima")
    n_pages, page_size = rows.shape[0], rows.shape[1]
    L = lib()
    if latent_attention_uses_tensor_cores(H, R, q.dtype):
        _check(L.pllm_latent_attention_mma(_ptr(q), _ptr(rows), _ptr(block_tables), _ptr(work), _ptr(n_work), max_work, _ptr(out),
                                           _ptr(part_o), _ptr(part_ml), H, R, page_size, n_pages, block_tables.shape[-1],
                                           float(scale), _ptr(status), _stream()), "latent_attention (mma)")
    else:
        _check(L.pllm_latent_attention_generic(_code(q), _ptr(q), _ptr(rows), _ptr(block_tables), _ptr(work), _ptr(n_work),
                                               max_work, _ptr(out), _ptr(part_o), _ptr(part_ml), H, R, page_size, n_pages,
                                               block_tables.shape[-1], float(scale), _ptr(status), _stream()),
               "latent_attention")
    _check(L.pllm_attention_reduce(_code(q), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red, _ptr(out), H, R,
                                   1 if (w.many_splits and R * 4 <= 1024) else 0, _stream()), "attention_reduce")
    return out


# ---- mixture of experts (csrc/moe.cu) -----------------------------------------------------------------------

ROUTER_SCORINGS = {"softmax": 0, "sigmoid": 1}
UNARY_KINDS = {"none": 0, "squared_relu": 1}      # one-argument activations of feed-forwards without a gate (common.cuh)


def _expert_act(act: str, gated: bool) -> int:
    if gated:
        return _glu(act)
    if act not in UNARY_KINDS:
        raise KernelError(f"activation {act!r} of experts without a gate is not known; known: {sorted(UNARY_KINDS)}")
    return UNARY_KINDS[act]


def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
              bias: Optional[torch.Tensor] = None, extra: int = 0, scoring: str = "softmax", renormalize: bool = True):
    """The router: (ids int32 [T, top], weights float32 [T, top]).  w_router float32 [outputs + extra, width].
    ``bias`` (float32 [outputs]) is added to the logits.  With ``extra`` the matrix carries that many further rows
    behind the router's, and their products with h come back as a third value, float32 [T, extra].  ``scoring``: "softmax"
    over all logits, or "sigmoid" of each; ``renormalize`` False: a chosen output's weight is its score itself."""
    if scoring not in ROUTER_SCORINGS:
        raise KernelError(f"moe_route: scoring {scoring!r} is not known; known: {sorted(ROUTER_SCORINGS)}")
    _dev(h, w_router, correction, bias)
    _f32(w_router, "w_router"); _f32(correction, "correction"); _f32(bias, "bias")
    T, W = h.shape
    E = w_router.shape[0] - int(extra)
    if w_router.shape[1] != W or E < 1 or any(t is not None and t.numel() != E for t in (correction, bias)):
        raise KernelError("moe_route: the router's weight, correction or bias does not fit")
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
    more = torch.empty((T, extra), dtype=torch.float32, device=h.device) if extra else None
    _check(lib().pllm_moe_route(_code(h), _ptr(h), _ptr(w_router), _ptr(correction), _ptr(ids), _ptr(weights), T, W, E,
                                int(top), int(groups), int(keep), _ptr(bias), int(extra), _ptr(more),
                                ROUTER_SCORINGS[scoring] | (0 if renormalize else 2), _stream()), "moe_route")
    return (ids, weights, more) if extra else (ids, weights)


def moe_experts_few(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gu: torch.Tensor, w_d: torch.Tensor,
                    shared: Optional[torch.Tensor], act: str = "silu", limit: float = 0.0,
                    shared_gate: Optional[torch.Tensor] = None, gated: bool = True, weight_input: bool = False) -> torch.Tensor:
    """sum_k weights[t, k] * expert_{ids[t, k]}(h[t]) (+ shared[t]); an id at or above the experts with tensors is the
    identity.  w_gu [experts, 2 ff, width] (gate rows, then up rows), w_d [experts, width, ff].  The weight-streaming form.
    ``act``, ``limit``: the experts' gated activation.  ``shared_gate`` (float32 [T]): shared[t] is multiplied by its sigmoid.
    ``gated`` False: experts down(act(up h)) with w_gu [experts, ff, width] and a one-argument ``act``.  ``weight_input``: the
    sum is over expert(weights[t, k] * h[t]) instead."""
    _dev(h, ids, weights, w_gu, w_d, shared, shared_gate)
    _i32(ids, "ids"); _f32(weights, "weights"); _f32(shared_gate, "shared_gate")
    if shared_gate is not None and shared_gate.numel() != h.shape[0]:
        raise KernelError("moe_experts_few: the shared expert's gate must hold one number a token")
    T, W = h.shape
    E, two_ff, _ = w_gu.shape
    ff, top = (two_ff // 2 if gated else two_ff), ids.shape[1]
    if w_gu.shape != (E, (2 if gated else 1) * ff, W) or w_d.shape != (E, W, ff) or w_gu.dtype != h.dtype or w_d.dtype != h.dtype:
        raise KernelError("moe_experts_few: expert weights do not fit")
    if shared is not None and (shared.shape != h.shape or shared.dtype != h.dtype):
        raise KernelError("moe_experts_few: the shared expert's output must have h's shape and dtype")
    acts = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    out = torch.empty_like(h)
    L = lib()
    _check(L.pllm_moe_pair_glu(_code(h), _ptr(h), _ptr(ids), _ptr(w_gu), _ptr(acts), T, W, ff, top, E, _expert_act(act, gated),
                               float(limit), 1 if gated else 0, _ptr(weights) if weight_input else None, _stream()), "moe_pair_glu")
    _check(L.pllm_moe_pair_down(_code(h), _ptr(acts), _ptr(h), _ptr(ids), _ptr(weights), _ptr(w_d), _ptr(shared), _ptr(out),
                                T, W, ff, top, E, _ptr(shared_gate), 1 if weight_input else 0, _stream()), "moe_pair_down")
    return out


# Many rows in bfloat16: the pairs sorted by expert and the tcgen05 product in its grouped form (csrc/gemm_tcgen05.cu).
# Below this many tokens a step's pairs are too few to fill tiles of 128 rows an expert, and the weight-streaming
# form reads less.
MOE_GROUPED_MIN_TOKENS = int(os.environ.get("PAGED_LLM_MOE_GROUPED_MIN", "48"))


def moe_grouped_takes(h: torch.Tensor, w_gu: torch.Tensor, w_d: torch.Tensor, gated: bool = True) -> bool:
    if h.dtype != torch.bfloat16 or h.shape[0] < MOE_GROUPED_MIN_TOKENS or TCGEN05_GEMM < 1:
        return False
    E, two_ff, W = w_gu.shape
    ff = two_ff // 2 if gated else two_ff
    L = lib()
    return bool(L.pllm_gemm_tcgen05_supports(128, ff, W, 1 if gated else 0)) and bool(L.pllm_gemm_tcgen05_supports(128, W, ff, 0))


def moe_experts_grouped(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gu: torch.Tensor, w_d: torch.Tensor,
                        shared: Optional[torch.Tensor], status: Optional[torch.Tensor] = None, act: str = "silu",
                        limit: float = 0.0, shared_gate: Optional[torch.Tensor] = None, gated: bool = True,
                        weight_input: bool = False) -> torch.Tensor:
    """The same sum as ``moe_experts_few`` by sorting the (token, expert) pairs by expert, two grouped tensor-core
    products (the first with the activation in its epilogue) and a weighted combine; with ``weight_input`` the gathered
    rows are multiplied by their weights instead."""
    _dev(h, ids, weights, w_gu, w_d, shared, shared_gate)
    _i32(ids, "ids"); _f32(weights, "weights"); _f32(shared_gate, "shared_gate")
    T, W = h.shape
    E, two_ff, _ = w_gu.shape
    ff, top = (two_ff // 2 if gated else two_ff), ids.shape[1]
    if not moe_grouped_takes(h, w_gu, w_d, gated) or w_gu.shape != (E, (2 if gated else 1) * ff, W) or w_d.shape != (E, W, ff):
        raise KernelError("moe_experts_grouped: shapes or dtypes the grouped product does not take")
    n_pairs = T * top
    max_tiles = -(-n_pairs // 128) + E
    slots = max_tiles * 128
    dev = h.device
    slot_pair = torch.empty(slots, dtype=torch.int32, device=dev)
    pair_slot = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    xs = torch.empty((slots, W), dtype=h.dtype, device=dev)
    acts = torch.empty((slots, ff), dtype=h.dtype, device=dev)
    y = torch.empty((slots, W), dtype=h.dtype, device=dev)
    out = torch.empty_like(h)
    st = status if status is not None else gemm_status(dev)
    L = lib()
    _check(L.pllm_moe_align(_ptr(ids), n_pairs, E, _ptr(slot_pair), _ptr(pair_slot), _ptr(tile_expert), max_tiles, _stream()),
           "moe_align")
    _check(L.pllm_moe_gather(_code(h), _ptr(h), _ptr(slot_pair), _ptr(tile_expert), _ptr(xs), slots, W, top,
                             _ptr(weights) if weight_input else None, _stream()), "moe_gather")
    _check(L.pllm_gemm_tcgen05_grouped(_ptr(xs), _ptr(w_gu), _ptr(acts), slots, ff, W,
                                       1 + _glu(act) if gated else -_expert_act(act, False), float(limit), _ptr(tile_expert),
                                       E, _ptr(st), _stream()), "gemm_tcgen05_grouped (gate/up)")
    _check(L.pllm_gemm_tcgen05_grouped(_ptr(acts), _ptr(w_d), _ptr(y), slots, W, ff, 0, 0.0, _ptr(tile_expert), E, _ptr(st), _stream()),
           "gemm_tcgen05_grouped (down)")
    _check(L.pllm_moe_combine(_code(h), _ptr(y), _ptr(h), _ptr(pair_slot), _ptr(weights), _ptr(shared), _ptr(out), T, W, top,
                              _ptr(shared_gate), 1 if weight_input else 0, _stream()), "moe_combine")
    return out


def moe_experts(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gu: torch.Tensor, w_d: torch.Tensor,
                shared: Optional[torch.Tensor], status: Optional[torch.Tensor] = None, act: str = "silu", limit: float = 0.0,
                shared_gate: Optional[torch.Tensor] = None, gated: bool = True, weight_input: bool = False) -> torch.Tensor:
    """The routed experts' weighted sum (+ the shared expert's output), by the form that fits the step."""
    if moe_grouped_takes(h, w_gu, w_d, gated):
        return moe_experts_grouped(h, ids, weights, w_gu, w_d, shared, status, act, limit, shared_gate, gated, weight_input)
    return moe_experts_few(h, ids, weights, w_gu, w_d, shared, act, limit, shared_gate, gated, weight_input)


# ---- a float32 stream with pre-norm blocks (csrc/stream32.cu) ----------------------------------------------------

def embed_norm32(tokens: torch.Tensor, table: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
                 status: torch.Tensor) -> torch.Tensor:
    """out[t] = rmsnorm(table[tokens[t]]) * gain as float32, whatever the table's dtype."""
    _dev(tokens, table, gain, out, status)
    _i32(tokens, "tokens"); _f32(out, "out"); _f32(gain, "gain")
    T, (V, H) = tokens.numel(), table.shape
    if out.shape != (T, H) or gain.numel() != H:
        raise KernelError(f"embed_norm32: out is {tuple(out.shape)}, expected {(T, H)}, with a gain of {H}")
    _check(lib().pllm_embed_norm32(_code(table), _ptr(tokens), _ptr(table), _ptr(gain), _ptr(out), T, H, V, float(eps),
                                   _ptr(status), _stream()), "embed_norm32")
    return out


def add_scaled_norm32(x: torch.Tensor, delta: Optional[torch.Tensor], mult: float, gain: torch.Tensor, eps: float,
                      out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x (float32, in place) += mult * delta where delta is given; out[i] = rmsnorm(x[r]) * gain, r = rows[i] or i.
    With ``rows`` the sum is formed for those rows only and x is left as it is."""
    _dev(x, delta, gain, out, rows)
    _f32(x, "x"); _f32(gain, "gain"); _i32(rows, "rows")
    W = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if gain.numel() != W or out.shape != (n, W) or (delta is not None and (delta.shape != x.shape or delta.dtype != out.dtype)):
        raise KernelError("add_scaled_norm32: out, gain or delta does not fit")
    _check(lib().pllm_add_scaled_norm32(_code(out), _ptr(x), _ptr(delta), float(mult), _ptr(gain), _ptr(out), _ptr(rows), n, W,
                                        float(eps), _stream()), "add_scaled_norm32")
    return out


def add_scaled32(x: torch.Tensor, delta: torch.Tensor, mult: float) -> torch.Tensor:
    """x (float32, in place) += mult * delta."""
    _dev(x, delta)
    _f32(x, "x")
    if delta.shape != x.shape:
        raise KernelError("add_scaled32: delta must have x's shape")
    _check(lib().pllm_add_scaled32(_code(delta), _ptr(x), _ptr(delta), float(mult), x.numel(), _stream()), "add_scaled32")
    return x


def scale32(x: torch.Tensor, c: float) -> torch.Tensor:
    """x (float32, in place) *= c."""
    _dev(x)
    _f32(x, "x")
    _check(lib().pllm_scale32(_ptr(x), float(c), x.numel(), _stream()), "scale32")
    return x


# ---- attention with a capped score, a window that keeps the first tokens, and a sink (csrc/attention_sink.cu) ------

def rope_mix_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, positions: torch.Tensor,
                      slots: Optional[torch.Tensor], kv_pool: Optional[torch.Tensor], v_first: Optional[torch.Tensor],
                      lam: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, dk: int, dv: int,
                      status: torch.Tensor) -> torch.Tensor:
    """qkv [T, heads dk + kv_heads (dk + dv)]: q and k rotated on their first ``rot`` entries (entry i with i + rot/2, the
    angle position * inv_freq[i] a float32 product), q to q_out [T, heads dk], k | v to row ``slots[t]`` of kv_pool
    [pages, kv_heads, page_size, dk + dv] (a negative slot, or no pool, writes nothing).  ``v_first``: a view
    [T, kv_heads dv] (rows may be strided) of an earlier layer's values; v <- (1 - lam) v + lam v_first, lam one float32
    on the device."""
    _dev(qkv, q_out, inv_freq, positions, slots, kv_pool, lam, status)
    _f32(inv_freq, "inv_freq"); _f32(lam, "lam"); _i32(positions, "positions"); _i32(slots, "slots")
    T = qkv.shape[0]
    if qkv.shape != (T, num_heads * dk + num_kv_heads * (dk + dv)) or q_out.numel() != T * num_heads * dk or q_out.dtype != qkv.dtype:
        raise KernelError("rope_mix_kv_write: qkv or q_out does not fit the head counts and sizes")
    if rot and (inv_freq is None or inv_freq.numel() * 2 != rot):
        raise KernelError("rope_mix_kv_write: inv_freq must hold rot / 2 frequencies")
    if positions.numel() < T or (slots is not None and slots.numel() < T):
        raise KernelError("rope_mix_kv_write: positions / slots shorter than the tokens")
    page_size, pool_rows = 1, 0
    if kv_pool is not None:
        if kv_pool.dim() != 4 or kv_pool.shape[1] != num_kv_heads or kv_pool.shape[3] != dk + dv or kv_pool.dtype != qkv.dtype:
            raise KernelError(f"rope_mix_kv_write: the pool must be [pages, {num_kv_heads}, page_size, {dk + dv}] of {qkv.dtype}")
        page_size, pool_rows = kv_pool.shape[2], kv_pool.shape[0] * kv_pool.shape[2]
    vf_stride = 0
    if v_first is not None:
        if not v_first.is_cuda or v_first.dtype != qkv.dtype or v_first.shape != (T, num_kv_heads * dv) or v_first.stride(1) != 1 \
                or lam is None:
            raise KernelError("rope_mix_kv_write: v_first must be [T, kv_heads dv] of qkv's dtype with unit inner stride, and lam given")
        vf_stride = v_first.stride(0)
    _check(lib().pllm_rope_mix_kv_write(_code(qkv), _ptr(qkv), qkv.shape[1], _ptr(q_out), _ptr(inv_freq), int(rot), _ptr(positions),
                                        _ptr(slots), _ptr(kv_pool), _ptr(v_first), vf_stride, _ptr(lam), T, num_heads, num_kv_heads,
                                        dk, dv, page_size, pool_rows, _ptr(status), _stream()), "rope_mix_kv_write")
    return q_out


# PAGED_LLM_SINK_MMA=0: the CUDA-core kernel everywhere (for comparisons)
SINK_MMA = os.environ.get("PAGED_LLM_SINK_MMA", "1") != "0"


def attention_sink_uses_tensor_cores(dtype: torch.dtype, num_heads: int, num_kv_heads: int, dk: int, dv: int) -> bool:
    """bfloat16 with key and value sizes of 32, 64 or 128: the mma.sync kernel; everything else (and float32) runs the
    CUDA-core kernel."""
    return SINK_MMA and dtype == torch.bfloat16 and bool(
        lib().pllm_attention_sink_mma_supports(_BF16, int(num_heads), int(num_kv_heads), int(dk), int(dv)))


def attention_sink_tile_tokens(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32, dk: int = 0, dv: int = 0) -> int:
    """The most query tokens one work item of ``attention_sink`` may hold, for the kernel it picks."""
    if attention_sink_uses_tensor_cores(dtype, num_heads, num_kv_heads, dk, dv):
        return int(lib().pllm_attention_sink_mma_tile_tokens(int(num_heads), int(num_kv_heads)))
    return int(lib().pllm_attention_sink_tile_tokens(int(num_heads), int(num_kv_heads)))


def attention_sink_ctas_per_item(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32, dk: int = 0, dv: int = 0) -> int:
    rows = 64 if attention_sink_uses_tensor_cores(dtype, num_heads, num_kv_heads, dk, dv) else 16
    return num_kv_heads * -(-(num_heads // num_kv_heads) // rows)


def attention_sink(q: torch.Tensor, kv_pool: torch.Tensor, block_tables: torch.Tensor, w, out: torch.Tensor,
                   sinks: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, dk: int, dv: int, window: int, keep_first: int,
                   scale: float, cap: float, status: torch.Tensor) -> torch.Tensor:
    """Attention of the step's tokens over rows [k | v] of the paged pool [pages, kv_heads, page_size, dk + dv]:
    score = cap tanh(scale q.k / cap) (cap 0: uncapped); key j is seen from position p when j <= p and (p - j < window or
    j < keep_first) (window 0: every j <= p); the softmax's denominator also holds exp(sinks[head]).  ``w`` is the group's
    ``AttentionWork``; then the reduction of split items.  q [T, heads, dk], out [T, heads, dv]."""
    work, n_work, max_work, red, n_red, max_red = w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red
    part_o, part_ml = w.part_o, w.part_ml
    _dev(q, kv_pool, block_tables, work, n_work, out, part_o, part_ml, red, n_red, sinks, status)
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml"); _f32(sinks, "sinks")
    T = q.shape[0]
    if kv_pool.dim() != 4 or kv_pool.shape[1] != num_kv_heads or kv_pool.shape[3] != dk + dv or kv_pool.dtype != q.dtype:
        raise KernelError(f"attention_sink: the pool must be [pages, {num_kv_heads}, page_size, {dk + dv}] of q's dtype")
    if q.numel() != T * num_heads * dk or out.numel() != T * num_heads * dv or out.dtype != q.dtype:
        raise KernelError("attention_sink: q must be [T, heads, dk] and out [T, heads, dv]")
    if part_o.shape[1:] != (num_heads, dv) or part_ml.shape[1:] != (num_heads, 2):
        raise KernelError("attention_sink: the scratch for partial results is not [rows, heads, dv] and [rows, heads, 2]")
    if sinks is not None and sinks.numel() != num_heads:
        raise KernelError("attention_sink: one sink a head")
    if work.numel() < max_work * 8 or red.numel() < max_red * 4:
        raise KernelError("attention_sink: work / red lists shorter than their maxima")
    n_pages, page_size = kv_pool.shape[0], kv_pool.shape[2]
    L = lib()
    if attention_sink_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, dk, dv):
        _check(L.pllm_attention_sink_mma(_ptr(q), _ptr(kv_pool), _ptr(block_tables), _ptr(work), _ptr(n_work), max_work, _ptr(out),
                                         _ptr(part_o), _ptr(part_ml), _ptr(sinks), num_heads, num_kv_heads, dk, dv, page_size, n_pages,
                                         block_tables.shape[-1], int(window), int(keep_first), float(scale), float(cap), _ptr(status),
                                         _stream()), "attention_sink (mma)")
    else:
        _check(L.pllm_attention_sink(_code(q), _ptr(q), _ptr(kv_pool), _ptr(block_tables), _ptr(work), _ptr(n_work), max_work,
                                     _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(sinks), num_heads, num_kv_heads, dk, dv, page_size,
                                     n_pages, block_tables.shape[-1], int(window), int(keep_first), float(scale), float(cap),
                                     _ptr(status), _stream()), "attention_sink")
    _check(L.pllm_attention_reduce(_code(q), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red, _ptr(out), num_heads, dv,
                                   1 if (w.many_splits and dv * 4 <= 1024) else 0, _stream()), "attention_reduce")
    return out


# ---- the Mamba-2 mixer between its projections (csrc/mamba2.cu) ------------------------------------------------------

def mamba2_state_floats(heads: int, groups: int, vdim: int, state: int, taps: int) -> int:
    """Floats of a request's state slot: every head's state matrix, then each channel's last taps - 1 inputs."""
    return heads * state * vdim + (taps - 1) * (heads * vdim + 2 * groups * state)


def mamba2_mix(u: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
               d_skip: torch.Tensor, gain: torch.Tensor, segments: torch.Tensor, max_segment_tokens: int, state: torch.Tensor,
               out: torch.Tensor, heads: int, groups: int, vdim: int, n_state: int, taps: int, norm_groups: int,
               eps: float) -> torch.Tensor:
    """From the input projection's u [T, 2 inner + 2 groups n_state + heads] to the output projection's input
    [T, inner]: convolution and silu, the recurrence over each segment's tokens from and into its state slot, the gate
    and the grouped norm.  ``segments`` int32 [n, 4] on the device: first token, tokens, tokens before, state slot."""
    _dev(u, conv_w, conv_b, dt_bias, a_log, d_skip, gain, segments, state, out)
    for t, n in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip"), (gain, "gain"), (state, "state")):
        _f32(t, n)
    _i32(segments, "segments")
    T = u.shape[0]
    inner, channels = heads * vdim, heads * vdim + 2 * groups * n_state
    if u.shape != (T, inner + channels + heads) or out.shape != (T, inner) or out.dtype != u.dtype:
        raise KernelError("mamba2_mix: u must be [T, 2 inner + 2 groups state + heads] and out [T, inner] of one dtype")
    if conv_w.shape != (channels, taps) or conv_b.numel() != channels or conv_w.dtype != u.dtype or conv_b.dtype != u.dtype:
        raise KernelError("mamba2_mix: the convolution's taps must be [channels, taps] and its bias [channels], of u's dtype")
    if min(dt_bias.numel(), a_log.numel(), d_skip.numel()) != heads or gain.numel() != inner:
        raise KernelError("mamba2_mix: one dt_bias, A_log and D a head, and a gain of inner entries")
    if state.dim() != 2 or state.shape[1] < mamba2_state_floats(heads, groups, vdim, n_state, taps):
        raise KernelError("mamba2_mix: the state slots are too small")
    if segments.dim() != 2 or segments.shape[1] != 4:
        raise KernelError("mamba2_mix: segments must be [n, 4]")
    c_buf = torch.empty((T, channels), dtype=torch.float32, device=u.device)
    y_buf = torch.zeros((T, inner), dtype=torch.float32, device=u.device)      # (rows of no segment, a captured step's padding, stay zero)
    _check(lib().pllm_mamba2_mix(_code(u), _ptr(u), _ptr(conv_w), _ptr(conv_b), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(gain),
                                 _ptr(segments), segments.shape[0], int(max_segment_tokens), _ptr(state), state.stride(0),
                                 _ptr(c_buf), _ptr(y_buf), _ptr(out), T, heads, groups, vdim, n_state, taps, norm_groups,
                                 float(eps), _stream()), "mamba2_mix", launches=3)
    return out


# ---- a block that norms each sublayer's input and output, on a float32 stream (csrc/stream32.cu) ---------------------------

def sandwich_norm32(x: torch.Tensor, a: Optional[torch.Tensor], a_bias: Optional[torch.Tensor], gain_a: Optional[torch.Tensor],
                    gain: Optional[torch.Tensor], out: Optional[torch.Tensor], eps: float,
                    rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x (float32, in place) += norm(a + a_bias) * gain_a where a is given (a sublayer's output, normed before it is added);
    out[i] = norm(x[r]) * gain where out is given (the next sublayer's input), r = rows[i] or i.  With ``rows`` the sum is
    formed for those rows only and x is left as it is."""
    _dev(x, a, a_bias, gain_a, gain, out, rows)
    _f32(x, "x"); _f32(gain, "gain"); _f32(gain_a, "gain_a"); _f32(a_bias, "a_bias"); _i32(rows, "rows")
    W = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if a is not None and (a.shape != x.shape or gain_a is None or gain_a.numel() != W or (a_bias is not None and a_bias.numel() != W)):
        raise KernelError("sandwich_norm32: a must have x's shape, with a gain (and a bias, if any) of its width")
    if out is not None and (out.shape != (n, W) or gain is None or gain.numel() != W or (a is not None and a.dtype != out.dtype)):
        raise KernelError("sandwich_norm32: out or its gain does not fit")
    if a is None and out is None:
        return None
    dtype = out.dtype if out is not None else a.dtype
    _check(lib().pllm_sandwich_norm32(_code_of(dtype), _ptr(x), _ptr(a), _ptr(a_bias), _ptr(gain_a), _ptr(gain), _ptr(out), _ptr(rows),
                                      n, W, float(eps), _stream()), "sandwich_norm32")
    return out


def swiglu_bias(gate_up: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """out[n, I] = act(gate_up[n, :I] + bias[:I], gate_up[n, I:] + bias[I:]); bias float32 [2 I]."""
    _dev(gate_up, bias, out)
    _f32(bias, "bias")
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype or bias.numel() != two_i:
        raise KernelError("swiglu_bias: out must be [n, I] and bias [2 I] for an input [n, 2I] of out's dtype")
    _check(lib().pllm_swiglu_bias(_code(gate_up), _ptr(gate_up), _ptr(bias), _ptr(out), n, two_i // 2, _glu(act), float(limit),
                                  _stream()), "swiglu_bias")
    return out


def scaled_sum2(x: torch.Tensor, y: torch.Tensor, a: float, b: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a * x + b * y, formed in float and rounded once; ``out`` may be x or y (default: x)."""
    out = x if out is None else out
    _dev(x, y, out)
    if y.shape != x.shape or y.dtype != x.dtype or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("scaled_sum2: x, y and out must share one shape and dtype")
    _check(lib().pllm_scaled_sum2(_code(x), _ptr(x), _ptr(y), float(a), float(b), _ptr(out), x.numel(), _stream()), "scaled_sum2")
    return out


# ---- queries and keys that are normed before the attention, and a gate behind it (csrc/normed_qk.cu) ---------------------------

QK_NORMS = {None: 0, "head": 1, "projection": 2}


def normed_qk_kv_write(proj: torch.Tensor, k_off: int, v_off: int, q_out: torch.Tensor, q_gain: Optional[torch.Tensor],
                       k_gain: Optional[torch.Tensor], norm: Optional[str], eps: float, temp_coef: float, temp_every: int,
                       inv_freq: Optional[torch.Tensor], rot: int, positions: torch.Tensor, slots: Optional[torch.Tensor],
                       kv_pool: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, dk: int, dv: int, values_are_keys: bool,
                       status: torch.Tensor) -> torch.Tensor:
    """From a stacked projection ``proj`` [T, width] (q at 0, k at k_off, v at v_off) to the attention's inputs: q and k normed
    (``norm``: None, "head": each head by its own root mean square with one gain of dk entries, "projection": all heads at
    once with a gain of the projection's size), q times 1 + temp_coef ln(floor((p + 1) / temp_every) + 1) (temp_every 0:
    not), both rotated on the first ``rot`` entries of each head; q to q_out [T, heads dk], k | v to row ``slots[t]`` of
    kv_pool [pages, kv_heads, page_size, dk + dv].  ``values_are_keys``: v is the raw key projection (neither normed nor rotated)."""
    _dev(proj, q_out, q_gain, k_gain, inv_freq, positions, slots, kv_pool, status)
    _f32(q_gain, "q_gain"); _f32(k_gain, "k_gain"); _f32(inv_freq, "inv_freq"); _i32(positions, "positions"); _i32(slots, "slots")
    T, width = proj.shape
    if norm not in QK_NORMS:
        raise KernelError(f"normed_qk_kv_write: norm {norm!r} is not known; known: {list(QK_NORMS)}")
    if k_off + num_kv_heads * dk > width or (not values_are_keys and v_off + num_kv_heads * dv > width) or num_heads * dk > width:
        raise KernelError("normed_qk_kv_write: the projection is narrower than its parts")
    if q_out.numel() != T * num_heads * dk or q_out.dtype != proj.dtype:
        raise KernelError("normed_qk_kv_write: q_out does not fit")
    n_gain = {None: (0, 0), "head": (dk, dk), "projection": (num_heads * dk, num_kv_heads * dk)}[norm]
    if norm is not None and (q_gain is None or k_gain is None or q_gain.numel() != n_gain[0] or k_gain.numel() != n_gain[1]):
        raise KernelError("normed_qk_kv_write: the gains do not fit the norm")
    if rot and (inv_freq is None or inv_freq.numel() * 2 != rot):
        raise KernelError("normed_qk_kv_write: inv_freq must hold rot / 2 frequencies")
    if positions.numel() < T or (slots is not None and slots.numel() < T):
        raise KernelError("normed_qk_kv_write: positions / slots shorter than the tokens")
    page_size, pool_rows = 1, 0
    if kv_pool is not None:
        if kv_pool.dim() != 4 or kv_pool.shape[1] != num_kv_heads or kv_pool.shape[3] != dk + dv or kv_pool.dtype != proj.dtype:
            raise KernelError(f"normed_qk_kv_write: the pool must be [pages, {num_kv_heads}, page_size, {dk + dv}] of {proj.dtype}")
        page_size, pool_rows = kv_pool.shape[2], kv_pool.shape[0] * kv_pool.shape[2]
    _check(lib().pllm_normed_qk_kv_write(_code(proj), _ptr(proj), width, int(k_off), int(v_off), _ptr(q_out), _ptr(q_gain), _ptr(k_gain),
                                         QK_NORMS[norm], float(eps), float(temp_coef), int(temp_every), _ptr(inv_freq), int(rot),
                                         _ptr(positions), _ptr(slots), _ptr(kv_pool), T, num_heads, num_kv_heads, dk, dv,
                                         1 if values_are_keys else 0, page_size, pool_rows, _ptr(status), _stream()),
           "normed_qk_kv_write")
    return q_out


GATE_KINDS = {"sigmoid": 0, "silu": 1}


def gate_mul(y: torch.Tensor, gate: torch.Tensor, kind: str = "sigmoid", per: int = 1) -> torch.Tensor:
    """y[t, c] *= sigmoid(gate[t, c // per]) (or silu), in place; ``gate`` may be a column range of a wider tensor.
    ``per`` 1: a gate an entry; a head's size: a gate a head."""
    _dev(y)
    if kind not in GATE_KINDS:
        raise KernelError(f"gate_mul: kind {kind!r} is not known; known: {sorted(GATE_KINDS)}")
    if y.dim() != 2 or per < 1 or y.shape[1] % per or not gate.is_cuda or gate.shape != (y.shape[0], y.shape[1] // per) \
            or gate.dtype != y.dtype or gate.stride(1) != 1:
        raise KernelError("gate_mul: the gate must have y's rows and dtype, one entry for every ``per`` of y's, with unit inner stride")
    _check(lib().pllm_gate_mul(_code(y), _ptr(y), _ptr(gate), gate.stride(0), y.shape[0], y.shape[1], GATE_KINDS[kind], int(per),
                               _stream()), "gate_mul")
    return y


# ---- recurrent mixers with a matrix of state a head (csrc/matrix_memory.cu) ----------------------------------------------------

def mlstm_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of a request's state slot: every head's matrix, its normaliser vector and its running maximum."""
    return heads * dim * vdim + heads * dim + heads


def delta_state_floats(heads: int, kv_heads: int, dim: int, vdim: int, taps: int) -> int:
    """Floats of a request's state slot: every head's matrix, then each channel's last taps - 1 inputs."""
    return heads * dim * vdim + (taps - 1) * (2 * kv_heads * dim + heads * vdim)


def _segments_ok(segments: torch.Tensor, what: str):
    _i32(segments, "segments")
    if segments.dim() != 2 or segments.shape[1] != 4:
        raise KernelError(f"{what}: segments must be [n, 4]")


def mlstm_mix(u: torch.Tensor, gates: torch.Tensor, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float, gain: torch.Tensor,
              segments: torch.Tensor, state: torch.Tensor, out: torch.Tensor, heads: int, dim: int, vdim: int, eps: float,
              max_segment_tokens: int = 0) -> torch.Tensor:
    """From the input projection's u [T, heads (2 dim + 2 vdim)] = [q | k | v | gate] and the gates' float32 projection
    [T, 2 heads] = [i | f] to the output projection's input [T, heads vdim]: the matrix memory's recurrence over each
    segment's tokens from and into its state slot, each head over its root mean square, the gain, sigmoid(gate).
    max_segment_tokens bounds a segment's tokens where the caller knows it (a step of decoded tokens fetches fewer at a time)."""
    _dev(u, gates, i_bias, f_bias, gain, segments, state, out)
    for t, n in ((gates, "gates"), (i_bias, "i_bias"), (f_bias, "f_bias"), (gain, "gain"), (state, "state")):
        _f32(t, n)
    _segments_ok(segments, "mlstm_mix")
    T = u.shape[0]
    if u.shape != (T, heads * (2 * dim + 2 * vdim)) or out.shape != (T, heads * vdim) or out.dtype != u.dtype:
        raise KernelError("mlstm_mix: u must be [T, heads (2 dim + 2 vdim)] and out [T, heads vdim] of one dtype")
    if gates.shape != (T, 2 * heads) or min(i_bias.numel(), f_bias.numel()) != heads or gain.numel() != heads * vdim:
        raise KernelError("mlstm_mix: gates must be [T, 2 heads], with a bias a head and gate, and a gain of heads vdim entries")
    if state.dim() != 2 or state.shape[1] < mlstm_state_floats(heads, dim, vdim):
        raise KernelError("mlstm_mix: the state slots are too small")
    y_buf = torch.zeros((T, heads * vdim), dtype=torch.float32, device=u.device)     # (rows of no segment stay zero)
    dn_buf = torch.zeros((T, heads, 2), dtype=torch.float32, device=u.device)
    nm_buf = torch.empty((segments.shape[0], heads, dim + 1), dtype=torch.float32, device=u.device)
    _check(lib().pllm_mlstm_mix(_code(u), _ptr(u), u.shape[1], _ptr(gates), _ptr(i_bias), _ptr(f_bias), float(cap), _ptr(gain),
                                _ptr(segments), segments.shape[0], int(max_segment_tokens), _ptr(state), state.stride(0), _ptr(nm_buf),
                                _ptr(dn_buf), _ptr(y_buf), _ptr(out), T, heads, dim, vdim, float(eps), _stream()),
           "mlstm_mix", launches=3)
    return out


def delta_mix(u: torch.Tensor, conv_w: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, gain: torch.Tensor,
              segments: torch.Tensor, max_segment_tokens: int, state: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int,
              dim: int, vdim: int, taps: int, eps: float) -> torch.Tensor:
    """From the input projection's u [T, 2 kv_heads dim + 2 heads vdim] = [q | k | v | gate] and the float32 projection
    ba [T, 2 heads] = [b | a] to the output projection's input [T, heads vdim]: convolution and silu, unit q and k, the
    gated delta rule over each segment's tokens from and into its state slot, each head over its root mean square, the gain
    (vdim entries, shared by the heads), silu(gate)."""
    _dev(u, conv_w, ba, a_log, dt_bias, gain, segments, state, out)
    for t, n in ((ba, "ba"), (a_log, "a_log"), (dt_bias, "dt_bias"), (gain, "gain"), (state, "state")):
        _f32(t, n)
    _segments_ok(segments, "delta_mix")
    T = u.shape[0]
    channels = 2 * kv_heads * dim + heads * vdim
    if u.shape != (T, channels + heads * vdim) or out.shape != (T, heads * vdim) or out.dtype != u.dtype:
        raise KernelError("delta_mix: u must be [T, 2 kv_heads dim + 2 heads vdim] and out [T, heads vdim] of one dtype")
    if conv_w.shape != (channels, taps) or conv_w.dtype != u.dtype:
        raise KernelError("delta_mix: the convolution's taps must be [channels, taps] of u's dtype")
    if ba.shape != (T, 2 * heads) or min(a_log.numel(), dt_bias.numel()) != heads or gain.numel() != vdim:
        raise KernelError("delta_mix: ba must be [T, 2 heads], with one A_log and dt_bias a head, and a gain of vdim entries")
    if state.dim() != 2 or state.shape[1] < delta_state_floats(heads, kv_heads, dim, vdim, taps):
        raise KernelError("delta_mix: the state slots are too small")
    c_buf = torch.empty((T, channels), dtype=torch.float32, device=u.device)
    y_buf = torch.zeros((T, heads * vdim), dtype=torch.float32, device=u.device)     # (rows of no segment stay zero)
    _check(lib().pllm_delta_mix(_code(u), _ptr(u), u.shape[1], _ptr(conv_w), _ptr(ba), _ptr(a_log), _ptr(dt_bias), _ptr(gain),
                                _ptr(segments), segments.shape[0], int(max_segment_tokens), _ptr(state), state.stride(0), _ptr(c_buf),
                                _ptr(y_buf), _ptr(out), T, heads, kv_heads, dim, vdim, taps, float(eps), _stream()),
           "delta_mix", launches=3)
    return out


# ---- feed-forwards without a gate (csrc/elementwise.cu, csrc/gemm_tcgen05.cu) ---------------------------------------------

def unary_act(x: torch.Tensor, act: str) -> torch.Tensor:
    """x = act(x) in place, for a one-argument activation of ``UNARY_KINDS``."""
    _dev(x)
    if act not in UNARY_KINDS:
        raise KernelError(f"unary_act: activation {act!r} is not known; known: {sorted(UNARY_KINDS)}")
    if not x.is_contiguous():
        raise KernelError("unary_act: x must be contiguous")
    _check(lib().pllm_unary_act(_code(x), _ptr(x), x.numel(), UNARY_KINDS[act], _stream()), "unary_act")
    return x


def linear_act(x: torch.Tensor, weight: torch.Tensor, act: str, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x W^T) for a one-argument activation: the first half of a feed-forward without a gate.  In bfloat16 the
    activation sits in the epilogue of the weight-streaming product (few rows) or of the tcgen05 product (many rows);
    otherwise the product, then the activation in place."""
    if act not in UNARY_KINDS:
        raise KernelError(f"linear_act: activation {act!r} is not known; known: {sorted(UNARY_KINDS)}")
    N, K = weight.shape
    if x.shape[-1] != K:
        raise KernelError(f"linear_act: input width {x.shape[-1]} does not fit a weight of {tuple(weight.shape)}")
    if skinny_gemm_takes(x, weight, K) and N <= SKINNY_MAX_N:
        _dev(x, weight)
        out = torch.empty((x.shape[0], N), dtype=torch.bfloat16, device=x.device)
        _check(lib().pllm_skinny_gemm_act(_ptr(x), _ptr(weight), _ptr(out), x.shape[0], N, K, 0, UNARY_KINDS[act], _stream()),
               "skinny_gemm (activation)")
        return out
    if TCGEN05_GEMM >= 1 and x.shape[0] >= TCGEN05_MIN_M and gemm_tcgen05_takes(x, weight, N, False):
        _dev(x, weight)
        out = torch.empty((x.shape[0], N), dtype=torch.bfloat16, device=x.device)
        st = status if status is not None else gemm_status(x.device)
        _check(lib().pllm_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), x.shape[0], N, K, -UNARY_KINDS[act], 0.0, _ptr(st),
                                       _stream()), "gemm_tcgen05 (activation)")
        return out
    return unary_act(linear(x, weight, status=status), act)


# ---- differential attention and latent attention with a rotated key part (csrc/diff_attention.cu) -------------------------

def conv_state_floats(channels: int, taps: int) -> int:
    """Floats of a request's state slot for a short convolution: each channel's last taps - 1 inputs (at least one float)."""
    return max(1, (taps - 1) * channels)


def conv_rope_kv_write(proj: torch.Tensor, bias: Optional[torch.Tensor], conv_w: torch.Tensor, segments: torch.Tensor,
                       max_segment_tokens: int, state: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int,
                       positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor, kv_pool: Optional[torch.Tensor],
                       q_heads: int, k_heads: int, maps: int, dk: int, dv: int, status: torch.Tensor) -> torch.Tensor:
    """From a projection's [q | k | v] channels (the first columns of ``proj``) to the attention's inputs: + bias, a causal
    convolution of conv_w.shape[1] taps a channel over each segment's tokens (earlier inputs from the segment's state slot,
    which then takes this step's last ones), the first ``rot`` entries of each q and k head turned (entry i with i + rot / 2),
    q to ``q_out`` [T, q_heads dk], k | v to the token's rows of the joined pool [pages, k_heads, page_size, dk + dv].  With
    ``maps`` > 1 a kv head has that many keys a token, each a pool row of its own followed by the kv head's one value."""
    _dev(bias, conv_w, segments, state, inv_freq, positions, slots, q_out, kv_pool, status)
    if not proj.is_cuda:
        raise KernelError("conv_rope_kv_write: proj is not on a CUDA device")
    _segments_ok(segments, "conv_rope_kv_write")
    for t, n in ((bias, "bias"), (conv_w, "conv_w"), (state, "state"), (inv_freq, "inv_freq")):
        _f32(t, n)
    _i32(positions, "positions"); _i32(slots, "slots")
    T = proj.shape[0]
    channels = (q_heads + k_heads) * dk + (k_heads // maps) * dv
    taps = conv_w.shape[1]
    if proj.dim() != 2 or proj.shape[1] < channels or proj.stride(1) != 1 or conv_w.shape != (channels, taps) or not conv_w.is_contiguous():
        raise KernelError("conv_rope_kv_write: proj must hold the channels in its first columns, conv_w be [channels, taps]")
    if bias is not None and bias.numel() != channels:
        raise KernelError("conv_rope_kv_write: one bias a channel")
    if q_out.shape != (T, q_heads * dk) or q_out.dtype != proj.dtype or not q_out.is_contiguous():
        raise KernelError("conv_rope_kv_write: q_out must be [T, q_heads dk] of proj's dtype")
    if state.dim() != 2 or state.shape[1] < conv_state_floats(channels, taps):
        raise KernelError("conv_rope_kv_write: the state slots are too small")
    if rot and (inv_freq is None or inv_freq.numel() != rot // 2):
        raise KernelError("conv_rope_kv_write: one frequency for every rotated pair")
    pool_rows, page_size = 0, 1
    if kv_pool is not None:
        if kv_pool.dim() != 4 or kv_pool.shape[1] != k_heads or kv_pool.shape[3] != dk + dv or kv_pool.dtype != proj.dtype \
                or not kv_pool.is_contiguous():
            raise KernelError(f"conv_rope_kv_write: the pool must be [pages, {k_heads}, page_size, {dk + dv}] of proj's dtype")
        page_size, pool_rows = kv_pool.shape[2], kv_pool.shape[0] * kv_pool.shape[2]
    _check(lib().pllm_conv_rope_kv_write(_code(proj), _ptr(proj), proj.stride(0), _ptr(bias), _ptr(conv_w), taps, _ptr(segments),
                                         segments.shape[0], int(max_segment_tokens), _ptr(state), state.stride(0), _ptr(inv_freq),
                                         int(rot), _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(kv_pool), q_heads, k_heads, maps,
                                         dk, dv, page_size, pool_rows, _ptr(status), _stream()),
           "conv_rope_kv_write", launches=2 if taps > 1 else 1)
    return q_out


def diff_combine(a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, heads: int, group: int, dv: int, lam: float, post: float,
                 eps: float) -> torch.Tensor:
    """out[t, h] = post * sigmoid(gate[t, h]) * (a1 - lam a2) over its root mean square, for a [T, 2 heads, dv] whose heads are
    ordered [kv head][map][head of the group] (``group`` heads a kv head); ``gate`` [T, heads] may be a column range."""
    _dev(a, out)
    if not gate.is_cuda:
        raise KernelError("diff_combine: the gate is not on a CUDA device")
    T = a.shape[0]
    if a.numel() != T * 2 * heads * dv or out.shape != (T, heads * dv) or out.dtype != a.dtype or not a.is_contiguous():
        raise KernelError("diff_combine: a must be [T, 2 heads, dv] and out [T, heads dv] of one dtype")
    if gate.shape != (T, heads) or gate.dtype != a.dtype or gate.stride(1) != 1:
        raise KernelError("diff_combine: the gate must be [T, heads] of a's dtype with unit inner stride")
    _check(lib().pllm_diff_combine(_code(a), _ptr(a), _ptr(gate), gate.stride(0), _ptr(out), T, heads, group, dv, float(lam),
                                   float(post), float(eps), _stream()), "diff_combine")
    return out


def latent_rope_write(down: Optional[torch.Tensor], gain: Optional[torch.Tensor], eps: float, q: torch.Tensor, q_rows: torch.Tensor,
                      pool: Optional[torch.Tensor], slots: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                      heads: int, dim: int, rot_dim: int, rot: int, kv_rank: int, status: torch.Tensor,
                      row_out: Optional[torch.Tensor] = None, carried: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``down`` [T, kv_rank + rot_dim] (or None: no rows are made): the latent over its root mean square times ``gain`` and the
    key part with its first ``rot`` entries turned pairwise go side by side into the token's row of ``pool``
    [pages, page_size, kv_rank + rot_dim], and to ``row_out`` [T, kv_rank + rot_dim] if given.  Without ``down``, rows made
    that way earlier in the step (``carried``) are stored as they are.  ``q`` [T, heads (dim + rot_dim)] (may be a column range): each head's last
    rot_dim entries, turned likewise, go to the last rot_dim entries of ``q_rows`` [T, heads, kv_rank + rot_dim]."""
    _dev(gain, q_rows, pool, slots, positions, inv_freq, status, row_out, carried)
    if not q.is_cuda or (down is not None and not down.is_cuda):
        raise KernelError("latent_rope_write: q or down is not on a CUDA device")
    _f32(gain, "gain"); _f32(inv_freq, "inv_freq"); _i32(slots, "slots"); _i32(positions, "positions")
    T, width = q.shape[0], kv_rank + rot_dim
    for t, n in ((row_out, "row_out"), (carried, "carried")):
        if t is not None and (t.shape != (T, width) or t.dtype != q.dtype or not t.is_contiguous()):
            raise KernelError(f"latent_rope_write: {n} must be [T, kv_rank + rot_dim] of q's dtype")
    if down is not None and carried is not None:
        raise KernelError("latent_rope_write: rows are made from down or carried from an earlier layer, not both")
    if q.shape[1] != heads * (dim + rot_dim) or q.stride(1) != 1 or q_rows.shape != (T, heads, width) or not q_rows.is_contiguous() \
            or q_rows.dtype != q.dtype:
        raise KernelError("latent_rope_write: q must be [T, heads (dim + rot_dim)] and q_rows [T, heads, kv_rank + rot_dim]")
    if down is not None and (down.shape != (T, width) or down.stride(1) != 1 or down.dtype != q.dtype or gain is None or gain.numel() != kv_rank):
        raise KernelError("latent_rope_write: down must be [T, kv_rank + rot_dim] of q's dtype, with a gain of kv_rank entries")
    if rot and (inv_freq is None or inv_freq.numel() != rot // 2):
        raise KernelError("latent_rope_write: one frequency for every rotated pair")
    pool_rows = 0
    if pool is not None and (down is not None or carried is not None):
        if pool.dim() != 3 or pool.shape[2] != width or pool.dtype != q.dtype or not pool.is_contiguous():
            raise KernelError("latent_rope_write: the pool must be [pages, page_size, kv_rank + rot_dim] of q's dtype")
        pool_rows = pool.shape[0] * pool.shape[1]
    _check(lib().pllm_latent_rope_write(_code(q), _ptr(down), down.stride(0) if down is not None else 0, _ptr(gain), float(eps), _ptr(q),
                                        q.stride(0), _ptr(q_rows), _ptr(pool) if pool_rows else None, _ptr(row_out), _ptr(carried), _ptr(slots),
                                        _ptr(positions), _ptr(inv_freq), T, heads, dim, rot_dim, int(rot), kv_rank, pool_rows,
                                        _ptr(status), _stream()), "latent_rope_write")
    return q_rows
