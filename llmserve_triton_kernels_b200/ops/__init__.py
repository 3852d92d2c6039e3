"""The engine's device operations: thin, checked wrappers over the CUDA library.

Every function here launches hand-written sm_100a kernels from ``csrc/`` on the current CUDA
stream (the bfloat16 matrix products may go to the vendor's library, as the reference's do:
src/llmserve/model/llama.py:80-88, 120, 185 call ``F.linear``).  There is no CPU path: without
a CUDA device, or if the library cannot be built and loaded, the first call raises.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import build as _build

_F32, _BF16 = 0, 1
_lib = None
_lock = threading.Lock()

_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_SIGNATURES = {
    "llm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "llm_rmsnorm": [_vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "llm_rope_kv_write": [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "llm_swiglu": [_vp, _vp, _i, _i, _i, _vp, _vp],
    "llm_add_bias": [_vp, _i, _i, _i, _i, _vp, _vp],
    "llm_fetch_words": [_vp, _vp, _vp, _i, _i, _vp],
    "llm_set_error_flag": [_vp],
    "llm_check_step_arrays": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_check_page_group": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "llm_linear_decode": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _f, _i, _i, _vp, _vp, _vp, _vp, _f, _vp, _vp],
    "llm_linear_decode_qkv": [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _f, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_tcgen05": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "llm_gemm_tcgen05_fused": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp],
    "llm_gemm_tcgen05_parts": [_i],
    "llm_attention_generic": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
    "llm_attention_mma": [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "llm_attention_mma_routed": [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "llm_attention_tcgen05": [_vp, _i, _vp, _i, _vp, ctypes.c_longlong, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "llm_argmax": [_vp, _i, _i, _vp, _vp, _vp],
    "llm_group_rmsnorm": [_vp, _vp, _i, _f, _vp, _f, _i, _vp, _vp, _i, _i, _i, _vp],
    "llm_stream_inject": [_vp, _vp, _i, _f, _vp, _vp, _i, _i, _vp, _i, _i, _vp],
    "llm_unary": [_vp, _i, _vp, _i, _i, _i, _i, _i, _f, _vp],
    "llm_gate_mul": [_vp, _ll, _ll, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "llm_mingru_scan": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "llm_latent_prepare": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _i, _vp],
    "llm_merge_project_gate": [_vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "llm_merge_two_parts": [_vp, _ll, _ll, _vp, _vp, _ll, _ll, _vp, _vp, _ll, _ll, _i, _i, _i, _vp],
    "llm_unit_norm_kv_write": [_vp, _i, _i, _vp, _vp, _f, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "llm_attention_rows": [_vp, _ll, _ll, _i, _vp, _ll, _ll, _i, _vp, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _i, _i,
                           _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _ll, _i, _i, _f, _vp],
    "llm_attention_rows_mma": [_vp, _ll, _ll, _i, _vp, _ll, _ll, _i, _vp, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _i,
                               _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp, _i, _vp, _ll, _i, _vp, _vp, _vp, _ll, _i, _i, _f, _vp],
    "llm_gemm_simt_batched": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _vp],
    "llm_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "llm_sigmoid_attention": [_vp, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i,
                              _i, _i, _vp],
    "llm_sigmoid_attention_mma": [_vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i, _i, _vp],
    "llm_sigmoid_sum_parts": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "llm_qk_prepare": [_vp, _i, _i, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _f, _vp, _i, _vp, _f, _i, _i, _i, _i, _i, _vp],
    "llm_retention_scan": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp],
    "llm_head_norm_gate": [_vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _f, _i, _vp, _vp],
    "llm_embed_copies": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "llm_hyper_mix_norm": [_vp, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _i, _vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "llm_head_prepare": [_vp, _i, _i, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _f, _i, _vp, _i, _vp, _f, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp],
    "llm_short_conv": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "llm_row_rmsnorm": [_vp, _i, _i, _vp, _f, _vp, _i, _i, _i, _i, _vp],
    "llm_gated_scan": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _i, _vp, _f, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp],
    "llm_expert_gated_act": [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _f, _f, _vp],
    "llm_router": [_vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "llm_route_topk": [_vp, _i, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp],
    "llm_expert_act_scale": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "llm_branch_sum_norm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _f, _f, _f, _vp],
    "llm_branch_norm_sum": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _f, _f, _vp],
}


class KernelError(RuntimeError):
    pass


def library():
    """The loaded CUDA library; built first if it is missing or out of date."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not torch.cuda.is_available():
                raise KernelError(
                    "no CUDA device is visible: this engine has no CPU path (its kernels are sm_100a CUDA)"
                )
            path = _build.build()
            lib = ctypes.CDLL(str(path))
            for name, args in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = args
                fn.restype = ctypes.c_int
            lib.llm_error_string.argtypes = [ctypes.c_int]
            lib.llm_error_string.restype = ctypes.c_char_p
            _lib = lib
            if torch.cuda.is_available():
                lib.llm_set_error_flag(_error_flag_ptr())  # for kernels whose entry points take no flag of their own
    return _lib


_launches = 0
_MMA_HEAD_DIMS = (16, 32, 64, 128)  # head sizes of the tensor-core attention; others take the general kernel
_SMALL_ROWS = 16  # requests with at most this many (token, group member) rows take the split-key shape
_SMALL_TILE_KEYS = 128  # keys one CTA of that shape covers per tile
_SPLIT_SCRATCH_BYTES = 16 << 20  # most scratch memory the split-key attention's partial results may take per call
_TC_ATTENTION_ENABLED = True
_TC_ATTENTION_HEAD_DIMS = (64, 128)
_TC_ATTENTION_PAGE_SIZES = (8, 16, 32, 64)
_TC_ATTENTION_MIN_TOKENS = 128  # a request with at least this many tokens in the step: attention on tcgen05
_TCGEN05_MIN_ROWS = 128  # from this many rows a bfloat16 product runs on tcgen05 with TMA-fed tiles (own kernel)
_DECODE_LINEAR_MAX_ROWS = 16  # up to this many rows a bfloat16 matrix product streams the weights once (own kernel)
_FORCE_GENERIC_ATTENTION = False  # tests switch the tensor-core attention off to reach the general kernel in bfloat16


_sm_counts: dict[int, int] = {}


def _sm_count() -> int:
    """SMs of the current device (asked once per device)."""
    device = torch.cuda.current_device()
    count = _sm_counts.get(device)
    if count is None:
        count = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


def launch_count() -> int:
    """How many kernels of the library have been launched by this process (a CUDA graph's replay
    counts the launches it captured)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _launch(name: str, *args) -> int:
    global _launches
    _launches += 1
    return getattr(library(), name)(*args)


def loaded_library_path() -> str | None:
    return None if _lib is None else _lib._name


def _check(code: int, what: str) -> None:
    if code != 0:
        text = _lib.llm_error_string(code).decode() if _lib is not None else ""
        raise KernelError(f"{what}: error {code} ({text})")


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {dtype} is not supported (float32 or bfloat16)")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked once per launch, so by the short way where torch has one (the Stream
    object of ``torch.cuda.current_stream()`` costs several microseconds to build)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous() and t.is_cuda, f"{name} must be a contiguous int32 CUDA tensor")


# ------------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, copies: int | None = None) -> torch.Tensor:
    """``float32(table[ids])``: ids ``[N]`` int32, table ``[vocab, hidden]`` -> ``[N, hidden]`` float32; with ``copies``
    the rows are written that many times, ``[copies, N, hidden]`` (a residual stream kept in several copies)."""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "the token table must be a contiguous matrix")
    n, (vocab, hidden) = ids.numel(), table.shape
    if copies is not None:
        out = torch.empty((int(copies), n, hidden), dtype=torch.float32, device=table.device)
        _check(_launch("llm_embed_copies", _ptr(ids), _ptr(table), _code(table.dtype), _ptr(out), n, hidden, vocab, int(copies), _stream()), "embed (copies)")
        return out
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(_launch("llm_embed", _ptr(ids), _ptr(table), _code(table.dtype), _ptr(out), n, hidden, vocab, _stream()), "embed")
    return out


def rmsnorm(
    resid: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    delta: torch.Tensor | None = None,
    rows: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """``v = resid (+ delta)``; returns ``v * rsqrt(mean(v^2) + eps) * weight`` in ``out_dtype``.
    Without ``rows`` the sum is written back to ``resid`` (float32, in place); with ``rows``
    (int32) only those rows are produced and ``resid`` is not changed."""
    _need(resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous(), "the residual must be a contiguous float32 matrix")
    _need(weight.dtype == torch.float32 and weight.numel() == resid.shape[1], "the norm weight must be float32 of the row size")
    if delta is not None:
        _need(delta.shape == resid.shape and delta.is_contiguous(), "delta must have the residual's shape")
    if rows is not None:
        _i32(rows, "rows")
    n_out = resid.shape[0] if rows is None else rows.numel()
    out = torch.empty((n_out, resid.shape[1]), dtype=out_dtype, device=resid.device)
    code = _launch("llm_rmsnorm", 
        _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else -1, _ptr(weight), float(eps),
        _ptr(rows), _ptr(out), _code(out_dtype), n_out, resid.shape[1], _stream(),
    )
    _check(code, "rmsnorm")
    return out


_error_flag: torch.Tensor | None = None


def _error_flag_ptr() -> int:
    """Address of a pinned host word that kernels set when one of their bounded waits gives up."""
    global _error_flag
    if _error_flag is None:
        _error_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_flag.data_ptr()


def check_device_errors() -> None:
    """Raise if a kernel reported that a bounded wait gave up, or (checked mode) that a step's arrays held an index out
    of its bounds (call after a synchronisation)."""
    if _error_flag is not None and int(_error_flag[0]) != 0:
        _error_flag[0] = 0
        raise KernelError("a kernel's wait for an asynchronous copy gave up; its results are not valid")
    if _check_status is not None and int(_check_status[0]) != 0:
        code, group, index, value, limit, count = (int(v) for v in _check_status[:6])
        _check_status.zero_()
        what = _CHECK_CODES.get(code, f"violation {code}")
        where = f" of page group {group}" if group >= 0 else ""
        raise KernelError(
            f"checked mode: {what}{where}: entry {index} holds {value} against {limit} ({count} violations in all); the entries were "
            "replaced by harmless ones before any kernel used them, and the step's results are not valid"
        )


# Checked mode (the environment variable LLMSERVE_B200_CHECKED=1, or set_checked): every step starts with kernels that
# look over its integer arrays on the device, where the step's kernels will read them (csrc/step_check.cu).
_checked = bool(os.environ.get("LLMSERVE_B200_CHECKED"))
_check_status: torch.Tensor | None = None
_CHECK_CODES = {
    1: "a token id outside the vocabulary", 2: "a position beyond the model's positions", 3: "a token that names a request it does not belong to",
    4: "token offsets that do not rise or do not end at the number of tokens", 5: "a context length shorter than the request's new tokens or beyond the model's positions",
    6: "a wanted row beyond the step's tokens", 7: "a state slot beyond the slots there are", 8: "a page table entry outside the pool",
    9: "a slot that is outside the pool or disagrees with the page table", 10: "a page table narrower than a request's pages",
}


def checked() -> bool:
    return _checked


def set_checked(on: bool) -> None:
    """Turn checked mode on or off for steps that run, or are captured as graphs, from now on."""
    global _checked
    _checked = bool(on)


def _check_status_ptr() -> int:
    global _check_status
    if _check_status is None:
        _check_status = torch.zeros(8, dtype=torch.int32).pin_memory()
    return _check_status.data_ptr()


def check_step_arrays(ctx, vocab: int, max_positions: int, state_slot_count: int = 0) -> None:
    """Checked mode: compare a step's token ids, positions, request indices, offsets, lengths, wanted rows and state
    slots with their limits on the device; a violation is recorded for :func:`check_device_errors` and repaired."""
    _check(_launch(
        "llm_check_step_arrays", _ptr(ctx.token_ids), _ptr(ctx.positions), _ptr(ctx.token_request), _ptr(ctx.cu_tokens),
        _ptr(ctx.context_lens), _ptr(ctx.logit_rows) if ctx.num_logits else None, _ptr(ctx.state_slots), ctx.num_tokens,
        ctx.num_requests, ctx.num_logits, vocab, max_positions, state_slot_count, _check_status_ptr(), _stream(),
    ), "check_step_arrays")


def check_page_group(ctx, page_table: torch.Tensor, slot_map: torch.Tensor, page_size: int, num_pages: int,
                     window: int | None, group: int) -> None:
    """Checked mode, after :func:`check_step_arrays`: every page table entry that the step may read lies inside the pool
    of ``num_pages`` pages, and every new token's slot is the one its page table gives."""
    _check(_launch(
        "llm_check_page_group", _ptr(page_table), page_table.shape[1], _ptr(slot_map), _ptr(ctx.positions), _ptr(ctx.token_request),
        _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), ctx.num_tokens, ctx.num_requests, page_size, num_pages, window or 0, group,
        _check_status_ptr(), _stream(),
    ), "check_page_group")


class NormedInput:
    """A normalised activation in factored form, as the fused decode kernels hand it on:
    ``xw [M, hidden]`` holds ``v * norm_weight`` (``v`` the residual stream after the last sum) and
    ``ss [parts, M]`` partial sums of ``v^2`` per row, so that
    ``normalised = xw * rsqrt(ss.sum(0) / hidden + eps)``.  ``ops.linear`` and ``ops.linear_swiglu``
    take it in place of a tensor and apply the row scale to their result; anything else calls
    :meth:`materialize`."""

    def __init__(self, xw: torch.Tensor, ss: torch.Tensor, eps: float, norm=None):
        self.xw, self.ss, self.eps, self.norm = xw, ss, float(eps), norm
        self.shape, self.dtype, self.device = xw.shape, xw.dtype, xw.device

    def materialize(self) -> torch.Tensor:
        scale = torch.rsqrt(self.ss.sum(0) / self.xw.shape[1] + self.eps)
        return (self.xw.float() * scale[:, None]).to(self.xw.dtype)


class _Added:
    """What :meth:`ResidualSink.linear` returns when the product has been added to the residual stream and nothing is
    left pending: the next norm normalises the stream as it stands."""

    def __repr__(self) -> str:
        return "ADDED"


ADDED = _Added()


class Scaled:
    """A contribution that enters the residual stream times ``alpha`` (layers that scale what their parts add)."""

    def __init__(self, tensor: torch.Tensor, alpha: float):
        self.tensor, self.alpha = tensor, float(alpha)


class BranchSum:
    """A contribution that is still a list of branch outputs: ``factor * sum_b rmsnorm(branches[b]) * weights[b]`` (what
    mixers side by side return).  A norm that knows it (``add_branches``) adds it to the stream and normalises in one
    kernel (:func:`branch_sum_rmsnorm`); anybody else gets the tensor from :meth:`materialize`."""

    def __init__(self, branches: list[torch.Tensor], weights: list[torch.Tensor], eps: float, factor: float):
        self.branches, self.weights, self.eps, self.factor = branches, weights, float(eps), float(factor)

    def materialize(self) -> torch.Tensor:
        return branch_norm_sum(self.branches, self.weights, self.eps, self.factor)


class WeightedSum:
    """A contribution that is still a list of tensors with a factor each: ``sum_b factors[b] * tensors[b]`` (what mixers
    side by side return when their outputs meet as a plain weighted sum).  Whoever takes it up in a kernel of its own
    (:func:`hyper_mix_norm`) reads the tensors; anybody else gets the sum from :meth:`materialize`."""

    def __init__(self, tensors: list[torch.Tensor], factors: list[float]):
        self.tensors, self.factors = list(tensors), [float(f) for f in factors]

    def materialize(self) -> torch.Tensor:
        out = unary(self.tensors[0].float() if self.tensors[0].dtype != torch.float32 else self.tensors[0], "scale", self.factors[0])
        for t, f in zip(self.tensors[1:], self.factors[1:]):
            out.add_(t.to(out.dtype), alpha=f)
        return out


class StreamUpdate:
    """What a part between hyper-connections returned, not yet taken up by the copies of the stream: ``result`` (a
    float32 tensor ``[N, width]`` or a :class:`WeightedSum`), and the part's ``mix [S, S]`` (from, to) and ``take [S]``:
    ``x_t <- sum_s mix[s, t] x_s + take[t] * result``."""

    def __init__(self, result, mix: torch.Tensor, take: torch.Tensor):
        self.result, self.mix, self.take = result, mix, take

    def results(self) -> tuple[list[torch.Tensor], list[float]]:
        if isinstance(self.result, WeightedSum):
            return self.result.tensors, self.result.factors
        if isinstance(self.result, Scaled):
            return [self.result.tensor], [self.result.alpha]
        if isinstance(self.result, BranchSum):
            return [self.result.materialize()], [1.0]
        return [self.result], [1.0]


def split_pending(pending) -> tuple[torch.Tensor | None, float]:
    """``(what is still to be added to the stream or None, its factor)`` of what a part or a block returned."""
    if isinstance(pending, (BranchSum, WeightedSum)):
        return pending.materialize(), 1.0
    if pending is None or pending is ADDED:
        return None, 1.0
    if isinstance(pending, Scaled):
        return pending.tensor, pending.alpha
    return pending, 1.0


class ResidualSink:
    """Where a part's last matrix product may put its result: added to the 32-bit residual stream ``resid`` in place.
    For few rows the fused decode kernel does it and hands the stream on normalised for ``norm`` (an RMS norm's
    ``weight`` and ``eps``; None: a norm that cannot be folded into a product's end) as a :class:`NormedInput`; for
    more rows the product's own epilogue adds into the stream (the library's product with the stream as its addend,
    accumulated and written in 32-bit), and :data:`ADDED` is returned: no contribution travels through memory to be
    added by the norm's kernel, which then only reads the stream.  Built by a block for bfloat16 steps."""

    def __init__(self, resid: torch.Tensor, weight: torch.Tensor | None, eps: float, norm=None, alpha: float = 1.0):
        """``alpha``: the product enters the stream times this (only the library's way takes a factor other than 1)."""
        self.resid, self.weight, self.eps, self.norm, self.alpha = resid, weight, float(eps), norm, float(alpha)

    @staticmethod
    def usable(num_tokens: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16

    def linear(self, x: torch.Tensor, w: torch.Tensor) -> "NormedInput | _Added | None":
        """``resid += x @ w^T``; returns the stream normalised for ``norm``, or :data:`ADDED`, or None if no way
        takes the operands (then nothing was changed)."""
        m, k = x.shape
        n = w.shape[0]
        if not (x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous() and self.resid.is_contiguous()):
            return None
        if m <= _DECODE_LINEAR_MAX_ROWS and self.weight is not None and self.alpha == 1.0:
            parts = -(-n // 16)
            xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
            ss = torch.empty((parts, m), dtype=torch.float32, device=x.device)
            code = _launch(
                "llm_linear_decode", _ptr(x), _ptr(w), None, _BF16, m, n, k, x.stride(0), n, None, 0, 0.0, 2, 0,
                _ptr(self.resid), _ptr(self.weight), _ptr(xw), _ptr(ss), 1.0, _error_flag_ptr(), _stream(),
            )
            if code != 10002:
                _check(code, "linear into the residual stream")
                return NormedInput(xw, ss, self.eps, self.norm)
            add_launches(-1)  # a shape the kernel refuses: the library's way below
        elif m <= _DECODE_LINEAR_MAX_ROWS:
            # the same kernel adds its product, times alpha, into the stream and leaves the norm to its own kernel
            code = _launch(
                "llm_linear_decode", _ptr(x), _ptr(w), None, _BF16, m, n, k, x.stride(0), n, None, 0, 0.0, 5, 0,
                _ptr(self.resid), None, None, None, self.alpha, _error_flag_ptr(), _stream(),
            )
            if code != 10002:
                _check(code, "linear into the residual stream (scaled)")
                return ADDED
            add_launches(-1)
        if _GEMM_POLICY == "own" and m >= _TCGEN05_MIN_ROWS:
            return None  # the caller runs the own tcgen05 product and leaves the sum to the norm's kernel
        library()
        torch.addmm(self.resid, x, w.t(), alpha=self.alpha, out_dtype=torch.float32, out=self.resid)
        return ADDED

    def linear_tcgen05(self, x: torch.Tensor, w: torch.Tensor) -> "NormedInput | None":
        """The same by the own tcgen05 kernel for 128 rows and more, whose four epilogue warps turn each 32 x 32 piece
        round in shared memory so that the 32-bit stream is read and written 128 bytes at a time.  Correct, and kept
        under test, but four warps per SM do not keep enough of the stream in flight: a prompt of 2,048 tokens on a
        1.1B model took 6.04 ms this way against 5.46 ms with the sum left to the norm's kernel, so no part calls it."""
        m, k = x.shape
        n = w.shape[0]
        if not (x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous() and m >= _TCGEN05_MIN_ROWS and self.weight is not None and self.alpha == 1.0):
            return None
        parts = library().llm_gemm_tcgen05_parts(n)
        xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        ss = torch.empty((parts, m), dtype=torch.float32, device=x.device)
        code = _launch(
            "llm_gemm_tcgen05_fused", _ptr(x), x.stride(0), _ptr(w), None, _BF16, m, n, k, n, 2, 0, None, 0, 0.0,
            _ptr(self.resid), _ptr(self.weight), _ptr(xw), _ptr(ss), _error_flag_ptr(), _stream(),
        )
        if code == 10002:
            add_launches(-1)
            return None
        _check(code, "linear into the residual stream (tcgen05)")
        return NormedInput(xw, ss, self.eps, self.norm)


def _decode_linear(x, w, out_dtype, mode: int, n_out: int, up_offset: int = 0):
    """The weight-streaming product for few rows; None if it refuses the shape."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and m <= _DECODE_LINEAR_MAX_ROWS and xt.stride(1) == 1 and w.is_contiguous()):
        return None
    out = torch.empty((m, n_out), dtype=out_dtype, device=xt.device)
    code = _launch(
        "llm_linear_decode", _ptr(xt), _ptr(w), _ptr(out), _code(out_dtype), m, n_out, k, xt.stride(0), n_out,
        _ptr(x.ss) if scaled else None, x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, mode, up_offset,
        None, None, None, None, 1.0, _error_flag_ptr(), _stream(),
    )
    if code == 10002:  # a shape the kernel refuses
        add_launches(-1)
        return None
    _check(code, "linear (decode)")
    return out


def linear(x, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T -> [M, N]``.  float32 operands run on the CUDA cores in true 32-bit
    (fixed summation order); bfloat16 operands accumulate in 32-bit on the tensor cores: up to 16 rows
    through the weight-streaming kernel, more through the vendor's library (or, where ``_GEMM_POLICY`` says so,
    the own tcgen05 kernel from 128 rows on).  ``x`` may be a :class:`NormedInput`."""
    if isinstance(x, NormedInput):
        if x.shape[0] >= _TCGEN05_MIN_ROWS:
            out = _tcgen05_linear(x, w, out_dtype or x.dtype, 0, w.shape[0])
        else:
            out = _decode_linear(x, w, out_dtype or x.dtype, 0, w.shape[0])
        return out if out is not None else linear(x.materialize(), w, out_dtype)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype, f"linear: operand types differ ({x.dtype}, {w.dtype})")
    _need(x.stride(1) == 1 and w.is_contiguous(), "linear: operands must have unit inner stride")
    out_dtype = out_dtype or x.dtype
    m, k = x.shape
    n = w.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        code = _launch("llm_gemm_simt", _ptr(x), _F32, _ptr(w), _F32, _ptr(out), _code(out_dtype), m, n, k, x.stride(0), k, n, _stream())
        _check(code, "linear (float32)")
        return out
    _need(x.dtype == torch.bfloat16, f"linear: element type {x.dtype} is not supported")
    if m <= _DECODE_LINEAR_MAX_ROWS:
        out = _decode_linear(x, w, out_dtype, 0, n)
        if out is not None:
            return out
    if m >= _TCGEN05_MIN_ROWS and not _library_is_faster("plain", m):
        out = _tcgen05_linear(x, w, out_dtype, 0, n)
        if out is not None:
            return out
    return _library_linear(x, w, out_dtype)


# Which of two ways a bfloat16 product of many rows takes: the own tcgen05 kernel or the vendor's library (as the
# reference's F.linear).  Measured on a B200 in graphs of back-to-back products of one shape (hidden 2048, feed-forward
# 5632; own / library in microseconds): 128 rows 13.9 / 5.3 (stacked projection), 30.8 / 9.5 (down); 2,048 rows 28.7 /
# 17.6, 17.0 / 14.5 (output), 36.2 / 31.8; 8,192 rows 87.8 / 58.6, 189.6 / 129.9: the library's tiles of 256 rows over
# two SMs need half the operand traffic per SM of the own kernel's 128-row tiles, and it splits small grids along k.
# Gate and up with SwiGLU in the product's end, against the library's product and an activation kernel: 52 / 45 at 1,024
# rows, 55 / 62 at 1,536, 72 / 85 at 2,048, 285 / 315 at 8,192.  So "auto" gives plain products to the library and the
# gated one to the own kernel from _SWIGLU_OWN_MIN_ROWS rows on; "own" and "library" force one way (also through the
# environment variable LLMSERVE_B200_GEMM; the tests run the own kernel at every shape).
_GEMM_POLICY = os.environ.get("LLMSERVE_B200_GEMM", "auto")
_SWIGLU_OWN_MIN_ROWS = 1536


def _library_is_faster(kind: str, m: int) -> bool:
    if _GEMM_POLICY != "auto":
        return _GEMM_POLICY == "library"
    return kind == "plain" or m < _SWIGLU_OWN_MIN_ROWS


def _library_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    library()  # the engine never runs without its kernels, even where a matrix product is the vendor's
    if out_dtype == torch.float32 and x.dtype == torch.bfloat16:
        return torch.mm(x, w.t(), out_dtype=torch.float32)  # the 32-bit sums as they are, not rounded on the way
    out = torch.matmul(x, w.t())
    return out if out_dtype == out.dtype else out.to(out_dtype)


def _tcgen05_linear(x, w, out_dtype, mode: int, n_out: int, up_offset: int = 0):
    """The tcgen05 + TMA product for many rows (``x`` a tensor or a :class:`NormedInput`); None if
    it refuses the shape."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and xt.stride(1) == 1 and w.is_contiguous()):
        return None
    out = torch.empty((m, n_out), dtype=out_dtype, device=xt.device)
    code = _launch(
        "llm_gemm_tcgen05_fused", _ptr(xt), xt.stride(0), _ptr(w), _ptr(out), _code(out_dtype), m, n_out, k, n_out, mode,
        up_offset, _ptr(x.ss) if scaled else None, x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, None, None, None,
        None, _error_flag_ptr(), _stream(),
    )
    if code == 10002:
        add_launches(-1)
        return None
    _check(code, "linear (tcgen05)")
    return out


def linear_qkv_rope(
    x,
    w_in: torch.Tensor,
    positions: torch.Tensor,
    table: torch.Tensor | None,
    slot_map: torch.Tensor | None,
    pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    write_kv: bool = True,
) -> torch.Tensor | None:
    """For few bfloat16 rows, one kernel instead of three: the stacked query/key/value projection,
    the rotary encoding of query and key heads, and the write of keys and values into their
    pages.  Returns the rotated queries ``[M, num_heads * head_dim]``, or None when the shape is
    not taken (the caller then runs the product, the rotation and the write one by one)."""
    scaled = isinstance(x, NormedInput)
    xt = x.xw if scaled else x
    m, k = xt.shape
    if not (xt.dtype == torch.bfloat16 and m <= _DECODE_LINEAR_MAX_ROWS and xt.stride(1) == 1 and w_in.is_contiguous()):
        return None
    if head_dim % 16 or (table is not None and (table.dtype != torch.float32 or table.shape[1] != head_dim)):
        return None
    kv = num_kv_heads if write_kv else 0
    _need(w_in.shape[0] == (num_heads + 2 * kv) * head_dim, "the stacked projection does not match the heads")
    if kv:
        _i32(slot_map, "slot_map")
        _need(pool.dtype == torch.bfloat16 and pool.is_contiguous() and tuple(pool.shape[1:3]) == (2, kv) and pool.shape[4] == head_dim, "the pool plane does not match the heads")
    q = torch.empty((m, num_heads * head_dim), dtype=torch.bfloat16, device=xt.device)
    code = _launch(
        "llm_linear_decode_qkv", _ptr(xt), _ptr(w_in), _ptr(q), m, k, xt.stride(0), _ptr(x.ss) if scaled else None,
        x.ss.shape[0] if scaled else 0, x.eps if scaled else 0.0, _ptr(positions), _ptr(table),
        table.shape[0] if table is not None else 0, _ptr(slot_map) if kv else None, _ptr(pool) if kv else None, num_heads, kv,
        head_dim, pool.shape[3] if kv else 1, _error_flag_ptr(), _stream(),
    )
    if code == 10002:
        add_launches(-1)
        return None
    _check(code, "linear_qkv_rope")
    return q


def linear_swiglu(x, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for ``w_gate_up = [gate rows | up rows]``: one kernel for
    few bfloat16 rows, else a product followed by the activation kernel."""
    inter = w_gate_up.shape[0] // 2
    xt = x.xw if isinstance(x, NormedInput) else x
    if xt.dtype == torch.bfloat16 and xt.shape[0] <= _DECODE_LINEAR_MAX_ROWS:
        out = _decode_linear(x, w_gate_up, torch.bfloat16, 1, inter, up_offset=inter)
        if out is not None:
            return out
    if xt.dtype == torch.bfloat16 and xt.shape[0] >= _TCGEN05_MIN_ROWS:
        scaled = isinstance(x, NormedInput)  # the factored form goes the own way: the library knows nothing of it
        if scaled or not _library_is_faster("swiglu", xt.shape[0]):
            out = _tcgen05_linear(x, w_gate_up, torch.bfloat16, 1, inter, up_offset=inter)
            if out is not None:
                return out
        if not scaled:
            return swiglu(_library_linear(x, w_gate_up, torch.bfloat16))
    return swiglu(linear(x, w_gate_up))


def rope_kv_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    table: torch.Tensor | None,
    slot_map: torch.Tensor | None,
    pool: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    write_kv: bool = True,
) -> None:
    """Rotate the query heads of each ``qkv`` row in place by its position's table row, and (with
    ``write_kv``) store the rotated key heads and the value heads at the row's slot of ``pool``
    ``[pages, 2, kv_heads, page_size, head_dim]``.  ``table`` None: no rotation."""
    n = qkv.shape[0]
    width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width, f"qkv rows must hold {width} elements")
    _i32(positions, "positions")
    table_rows = 0
    if table is not None:
        _need(table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] == head_dim, "the rotary table must be float32 [positions, head_dim]")
        table_rows = table.shape[0]
    page_size = 1
    if write_kv:
        _i32(slot_map, "slot_map")
        _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5, "the pool plane must be contiguous [pages, 2, kv_heads, page_size, head_dim] of the qkv type")
        _need(pool.shape[1] == 2 and pool.shape[2] == num_kv_heads and pool.shape[4] == head_dim, "the pool plane does not match the heads")
        page_size = pool.shape[3]
    code = _launch("llm_rope_kv_write", 
        _ptr(qkv), _code(qkv.dtype), qkv.stride(0), _ptr(positions), _ptr(table), table_rows, _ptr(slot_map),
        _ptr(pool), n, num_heads, num_kv_heads if write_kv else 0, head_dim, page_size, int(write_kv), _stream(),
    )
    _check(code, "rope_kv_write")


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """Rotate ``x [N, heads, head_dim]`` (a view with unit inner strides per head) in place."""
    if x.shape[1] == 0 or x.shape[0] == 0:
        return
    _need(x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == x.shape[2], "rope_inplace: x must be [N, heads, head_dim] with packed heads")
    flat = x.as_strided((x.shape[0], x.shape[1] * x.shape[2]), (x.stride(0), 1), x.storage_offset())
    rope_kv_write(flat, positions, table, None, None, x.shape[1], 0, x.shape[2], write_kv=False)


def paged_attention(
    qkv: torch.Tensor,
    pool: torch.Tensor,
    page_table: torch.Tensor,
    ctx,
    *,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int | None = None,
) -> torch.Tensor:
    """Attention of every new token over its request's cached keys and values.

    ``qkv`` rows start with the (already rotated) query heads; the new tokens' keys and values are
    already in ``pool``.  ``ctx`` gives ``token_request``, ``cu_tokens`` and ``context_lens``:
    the token at flat row t of request r stands at position
    ``context_lens[r] - (cu_tokens[r+1] - cu_tokens[r]) + (t - cu_tokens[r])`` and sees the keys
    at positions ``max(0, p - window + 1) .. p``.  Returns ``[N, num_heads * head_dim]``."""
    n = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= num_heads * head_dim, "qkv rows must start with the query heads")
    _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5, "the pool plane must be contiguous and of the query type")
    _need(tuple(pool.shape[1:3]) == (2, num_kv_heads) and pool.shape[4] == head_dim, "the pool plane does not match the heads")
    _need(1 <= head_dim <= 256, f"head_dim {head_dim} is not supported (up to 256)")
    _i32(page_table, "page_table")
    out = torch.empty((n, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if qkv.dtype == torch.bfloat16 and head_dim in _MMA_HEAD_DIMS and not _FORCE_GENERIC_ATTENTION:
        group = num_heads // num_kv_heads
        # requests that bring at least 128 tokens: 128-token tiles of one head on tcgen05 (head sizes 64 and 128, pages
        # of 8 to 64 keys); the others: rows of (token, group member) on mma.sync, 64 rows a tile or the split-key shape
        tc_min = 0
        if head_dim in _TC_ATTENTION_HEAD_DIMS and pool.shape[3] in _TC_ATTENTION_PAGE_SIZES and _TC_ATTENTION_ENABLED:
            tc_min = _TC_ATTENTION_MIN_TOKENS
        num_requests, tc_longest, small, max_rows_large, other_rows = _attention_route(ctx, group, tc_min)
        if tc_longest:
            code = _launch(
                "llm_attention_tcgen05", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), pool.shape[0],
                _ptr(page_table), page_table.shape[1], _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), num_requests, n, num_heads,
                num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), tc_min, tc_longest, _error_flag_ptr(),
                _stream(),
            )
            if code == 10002:  # the kernel does not take this layout: all requests go the other way
                add_launches(-1)
                tc_min = 0
                num_requests, tc_longest, small, max_rows_large, other_rows = _attention_route(ctx, group, 0)
            else:
                _check(code, "paged_attention (tcgen05)")
        if not other_rows:
            return out
        splits = 1
        if small:
            longest = getattr(ctx, "max_context_len", None) or int(ctx.context_lens.max())
            useful = -(-longest // _SMALL_TILE_KEYS)
            splits = max(1, min(useful, _sm_count() // (small * num_kv_heads), 32))  # one CTA per SM at most: all run at once
            # the partial results are indexed by token over the whole step: beside a long portion of a prompt the
            # decode tokens are not split so finely that the scratch memory grows past a few megabytes
            splits = min(splits, max(1, _SPLIT_SCRATCH_BYTES // (n * num_heads * head_dim * 4)))
        scratch_o = scratch_ml = counters = None
        if splits > 1:
            counters = _split_counters(qkv.device, num_requests * num_kv_heads)
            scratch_o = torch.empty((n * num_heads * splits * head_dim,), dtype=torch.float32, device=qkv.device)
            scratch_ml = torch.empty((n * num_heads * splits * 2,), dtype=torch.float32, device=qkv.device)
        code = _launch(
            "llm_attention_mma_routed", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), _ptr(page_table),
            page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), num_requests, n,
            num_heads, num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), max_rows_large,
            int(small > 0), splits, 1, _ptr(scratch_o), _ptr(scratch_ml), _ptr(counters), tc_min if tc_longest else 0, _stream(),
        )
        add_launches((max_rows_large > 0) + (small > 0) - 1)
        _check(code, "paged_attention (tensor cores)")
        return out
    code = _launch(
        "llm_attention_generic", _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(pool), _code(qkv.dtype),
        _ptr(page_table), page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens), n,
        num_heads, num_kv_heads, head_dim, pool.shape[3], int(window or 0), float(scale), _stream(),
    )
    _check(code, "paged_attention")
    return out


def _attention_route(ctx, group: int, tc_min: int) -> tuple[int, int, int, int, bool]:
    """Which kernels a step's requests go to, from how many tokens each brings: (requests, most tokens of a request
    that the tcgen05 kernel takes (0: none), requests of the split-key shape, most rows of a request of the 64-row
    shape (0: none), any request for the mma.sync kernels at all).  The same for every layer of a step, so it is
    worked out once and kept on the step's context."""
    kept = ctx.__dict__.setdefault("_attention_routes", {}) if hasattr(ctx, "__dict__") else {}
    route = kept.get((group, tc_min))
    if route is None:
        cu = getattr(ctx, "host_cu_tokens", None)
        if cu is None:
            cu = ctx.cu_tokens.tolist()
        lens = [b - a for a, b in zip(cu, cu[1:])]
        tc_longest = max((x for x in lens if tc_min and x >= tc_min), default=0)
        rows = [x * group for x in lens if not (tc_longest and x >= tc_min)]
        small = sum(1 for x in rows if x <= _SMALL_ROWS)
        max_rows_large = max((x for x in rows if x > _SMALL_ROWS), default=0)
        route = kept[(group, tc_min)] = (len(lens), tc_longest, small, max_rows_large, bool(rows))
    return route


_counters: dict = {}


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed int32 counters that the split-key attention uses and leaves zeroed; one buffer per
    device, made on first use (outside any graph capture: the first step of a shape runs eagerly)."""
    buf = _counters.get(device)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(max(n, 16384), dtype=torch.int32, device=device)
        _counters[device] = buf
    return buf


def swiglu(gate_up: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(gate_up[:, :I]) * gate_up[:, I:]`` computed in 32-bit -> ``[N, I]``.  ``bias`` (``[2 I]``, of the rows' type,
    laid out like a row): the two projections' biases, added in 32-bit on the way in."""
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0, "gate_up must be a contiguous [N, 2 I] matrix")
    _need(bias is None or (bias.dtype == gate_up.dtype and bias.is_contiguous() and bias.numel() == gate_up.shape[1]), "swiglu: the bias is [2 I] of the rows' type")
    n, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(_launch("llm_swiglu", _ptr(gate_up), _ptr(out), _code(gate_up.dtype), n, inter, _ptr(bias), _stream()), "swiglu")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x [N, C] += bias [C]`` in place (summed in 32-bit, rounded once); returns ``x``."""
    _need(x.dim() == 2 and x.stride(1) == 1 and bias.dim() == 1 and bias.numel() == x.shape[1] and bias.is_contiguous(),
          "add_bias: x [N, C] with unit inner stride and bias [C]")
    _need(bias.dtype == x.dtype, f"add_bias: the bias is {bias.dtype}, the rows are {x.dtype}")
    _check(_launch("llm_add_bias", _ptr(x), _code(x.dtype), x.shape[0], x.shape[1], x.stride(0), _ptr(bias), _stream()), "add_bias")
    return x


def fetch_words(host: torch.Tensor, dev: torch.Tensor, head: torch.Tensor | None = None) -> None:
    """``dev[:] = host`` for int32 arrays of one size, ``host`` in pinned host memory: the kernel reads the host's
    memory itself.  Where ``head`` (int32, on the device) is given, the first ``len(head)`` words come from it
    instead.  The host must leave ``host`` alone until the stream has passed this point."""
    _need(host.dtype == torch.int32 and dev.dtype == torch.int32 and host.numel() == dev.numel(), "two int32 arrays of one size")
    _need(host.is_pinned() and dev.is_cuda and host.is_contiguous() and dev.is_contiguous(), "from pinned host memory to the device")
    if head is not None:
        _need(head.dtype == torch.int32 and head.is_cuda and head.is_contiguous() and head.numel() <= dev.numel(), "head: int32 on the device")
    code = _launch("llm_fetch_words", _ptr(host), _ptr(dev), _ptr(head), 0 if head is None else head.numel(), host.numel(), _stream())
    _check(code, "fetch_words")


def _host_out(host_out: torch.Tensor | None, rows: int) -> int | None:
    if host_out is None:
        return None
    _need(host_out.dtype == torch.int32 and host_out.numel() == rows and host_out.is_pinned() and host_out.is_contiguous(),
          "host_out must be int32 [rows] in pinned host memory")
    return host_out.data_ptr()


def argmax(logits: torch.Tensor, host_out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of each row (the lowest index among equals) -> int32 ``[rows]``.  ``host_out``
    (int32 ``[rows]`` in pinned host memory) gets the same from the kernel itself, valid once the stream has
    passed this point."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous float32 matrix")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    _check(_launch("llm_argmax", _ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _host_out(host_out, logits.shape[0]), _stream()), "argmax")
    return out


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    seeds: torch.Tensor,
    counters: torch.Tensor,
    host_out: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token per row: argmax where ``temperature <= 0``, else a draw from
    ``softmax(logits / temperature)`` cut by ``top_k`` (0: off) and ``top_p`` (1: off) at the
    uniform number that ``(seed, counter)`` gives.  All parameter tensors are ``[rows]`` on the
    device: float32, int32, float32, int64, int64.  ``host_out``: as for ``argmax``."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous float32 matrix")
    rows = logits.shape[0]
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"), (top_p, torch.float32, "top_p"), (seeds, torch.int64, "seeds"), (counters, torch.int64, "counters")):
        _need(t.dtype == dt and t.numel() == rows and t.is_contiguous() and t.is_cuda, f"{name} must be {dt} [rows] on the device")
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    code = _launch("llm_sample", 
        _ptr(logits), rows, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seeds), _ptr(counters),
        _ptr(out), _host_out(host_out, rows), _stream(),
    )
    _check(code, "sample")
    return out


# ------------------------------------------------------------------------------------------------
# Operations of layers that normalise in groups, scale their contributions, gate their outputs, keep a recurrent
# state, or attend over a latent (csrc/stream_ops.cu, recurrent.cu, cache_write.cu, attention_generic.cu).
_UNARY_KINDS = {"relu2": 0, "gelu_tanh": 1, "scale": 2, "silu": 3}
_GATE_KINDS = {"sigmoid": 0, "silu": 1}


def group_rmsnorm(
    resid: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    groups: int,
    delta: torch.Tensor | None = None,
    alpha: float = 1.0,
    rows: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """``v = resid + alpha * delta``; each of ``groups`` equal consecutive parts of a row of ``v`` is divided by
    ``sqrt(mean(part^2) + eps)``; returns that times ``weight`` in ``out_dtype``.  Without ``rows`` the sum is written
    back to ``resid``; with ``rows`` (int32) only those rows are produced and ``resid`` is not changed."""
    _need(resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous(), "the residual must be a contiguous float32 matrix")
    _need(weight.dtype == torch.float32 and weight.numel() == resid.shape[1], "the norm weight must be float32 of the row size")
    _need(groups >= 1 and resid.shape[1] % groups == 0, f"rows of {resid.shape[1]} do not split into {groups} equal parts")
    if delta is not None:
        _need(delta.shape == resid.shape and delta.is_contiguous(), "delta must have the residual's shape")
    if rows is not None:
        _i32(rows, "rows")
    n_out = resid.shape[0] if rows is None else rows.numel()
    out = torch.empty((n_out, resid.shape[1]), dtype=out_dtype, device=resid.device)
    code = _launch(
        "llm_group_rmsnorm", _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else -1, float(alpha),
        _ptr(weight), float(eps), int(groups), _ptr(rows), _ptr(out), _code(out_dtype), n_out, resid.shape[1], _stream(),
    )
    _check(code, "group_rmsnorm")
    return out


def stream_inject(
    resid: torch.Tensor,
    delta: torch.Tensor | None = None,
    alpha: float = 1.0,
    ids: torch.Tensor | None = None,
    table: torch.Tensor | None = None,
    vector: torch.Tensor | None = None,
) -> None:
    """``resid[t] += alpha * delta[t] + float(table[ids[t]]) + vector`` in place, in that order, each addend optional:
    what a residual stream meets when a stretch of layers starts again."""
    _need(resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous(), "the residual must be a contiguous float32 matrix")
    n, hidden = resid.shape
    if delta is not None:
        _need(delta.shape == resid.shape and delta.is_contiguous(), "delta must have the residual's shape")
    if table is not None:
        _i32(ids, "ids")
        _need(table.dim() == 2 and table.is_contiguous() and table.shape[1] == hidden and ids.numel() == n, "the token table does not match the stream")
    if vector is not None:
        _need(vector.dtype == torch.float32 and vector.is_contiguous() and vector.numel() == hidden, "the vector must be float32 of the row size")
    code = _launch(
        "llm_stream_inject", _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else -1, float(alpha),
        _ptr(ids) if table is not None else None, _ptr(table), _code(table.dtype) if table is not None else -1,
        table.shape[0] if table is not None else 0, _ptr(vector), n, hidden, _stream(),
    )
    _check(code, "stream_inject")


def unary(x: torch.Tensor, kind: str, alpha: float = 1.0, inplace: bool = False) -> torch.Tensor:
    """A one-input function of every element, computed in 32-bit: ``relu2`` (the square of relu), ``gelu_tanh``,
    ``silu``, or ``scale`` (``alpha * x``).  ``x [N, C]`` may have a row pitch."""
    _need(kind in _UNARY_KINDS, f"no one-input function {kind!r}; known: {sorted(_UNARY_KINDS)}")
    _need(x.dim() == 2 and x.stride(1) == 1, "unary: a matrix with unit inner stride")
    out = x if inplace else torch.empty(x.shape, dtype=x.dtype, device=x.device)
    code = _launch("llm_unary", _ptr(x), x.stride(0), _ptr(out), out.stride(0), _code(x.dtype), x.shape[0], x.shape[1],
                   _UNARY_KINDS[kind], float(alpha), _stream())
    _check(code, "unary")
    return out


def linear_act(x, w: torch.Tensor, activation: str) -> torch.Tensor:
    """``act(x @ w^T)`` for a one-input activation (see :func:`unary`): the product, then the activation on its
    result in place; for few bfloat16 rows the square of relu is the end of the weight-streaming product itself."""
    xt = x.xw if isinstance(x, NormedInput) else x
    if activation == "relu2" and xt.dtype == torch.bfloat16 and xt.shape[0] <= _DECODE_LINEAR_MAX_ROWS:
        out = _decode_linear(x, w, torch.bfloat16, 4, w.shape[0])
        if out is not None:
            return out
    return unary(linear(x, w), activation, inplace=True)


def gate_mul(a: torch.Tensor, b: torch.Tensor, kind: str = "sigmoid", per_head: bool = False) -> torch.Tensor:
    """``a [N, heads, W]`` (any token and head strides) times ``gate(b [N, heads * W])`` -> ``[N, heads * W]``;
    the gate (``sigmoid`` or ``silu``) and the product are 32-bit.  ``per_head``: one gate a head, ``b [N, heads]``."""
    _need(kind in _GATE_KINDS, f"no gate {kind!r}; known: {sorted(_GATE_KINDS)}")
    _need(a.dim() == 3 and a.stride(2) == 1 and b.dim() == 2 and b.stride(1) == 1 and a.dtype == b.dtype, "gate_mul: a [N, heads, W], b [N, heads * W]")
    n, heads, w = a.shape
    _need(b.shape[0] == n and b.shape[1] == (heads if per_head else heads * w), "gate_mul: the gate does not match the heads")
    out = torch.empty((n, heads * w), dtype=a.dtype, device=a.device)
    code = _launch("llm_gate_mul", _ptr(a), a.stride(0), a.stride(1), w, _ptr(b), b.stride(0), _ptr(out), heads * w,
                   _code(a.dtype), n, heads * w, _GATE_KINDS[kind] | (2 if per_head else 0), _stream())
    _check(code, "gate_mul")
    return out


def mingru_scan(proj: torch.Tensor, bias_z, bias_u, states: torch.Tensor, state_slots: torch.Tensor, cu_tokens: torch.Tensor,
                num_requests: int, width: int, out_dtype: torch.dtype, max_query_len: int = 1 << 30) -> torch.Tensor:
    """The minGRU recurrence over a flat batch.  ``proj [N, 3 * width]`` holds the pre-activations of the update
    gate, the candidate and the output gate; ``states [slots, width]`` (float32) is read at ``state_slots[r]`` for
    request r, walked over the request's tokens ``cu_tokens[r]:cu_tokens[r+1]`` and written back.  ``max_query_len``:
    the most tokens a request brings (long requests are shared out over the warps of a CTA).  Returns
    ``state_t * silu(output gate)`` ``[N, width]`` in ``out_dtype``."""
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= 3 * width, "mingru_scan: proj rows hold three pre-activations")
    _need(states.dtype == torch.float32 and states.is_contiguous() and states.shape[1] == width, "mingru_scan: states must be float32 [slots, width]")
    for b in (bias_z, bias_u):
        _need(b is None or (b.dtype == torch.float32 and b.numel() == width and b.is_contiguous()), "mingru_scan: biases are float32 [width]")
    _i32(state_slots, "state_slots")
    _i32(cu_tokens, "cu_tokens")
    out = torch.empty((proj.shape[0], width), dtype=out_dtype, device=proj.device)
    code = _launch("llm_mingru_scan", _ptr(proj), _code(proj.dtype), proj.stride(0), _ptr(bias_z), _ptr(bias_u), _ptr(states),
                   _ptr(state_slots), _ptr(cu_tokens), _ptr(out), _code(out_dtype), width, int(num_requests), width, int(max_query_len), _stream())
    _check(code, "mingru_scan")
    return out


def latent_prepare(proj: torch.Tensor, positions: torch.Tensor, slot_map: torch.Tensor, plane: torch.Tensor, weight: torch.Tensor,
                   freq: torch.Tensor, eps: float, heads: int, dim: int, rot: int, rank: int, fresh: bool = False,
                   queries: torch.Tensor | None = None, kv_col: int = 0, halves: bool = False):
    """For latent attention, from a token's stacked projections ``proj`` = ``[heads x (dim | rot) | rank | rot | ...]``:
    the queries' rotated parts (interleaved pairs, angles ``position * freq[i]`` in 32-bit) are returned as
    ``[N, heads, rot]``; the latent, RMS-normed with ``weight``, and the rotated shared key part are written to the
    token's slot of ``plane [pages, page_size, rank + rot]``.  With ``fresh`` the written rows are also returned token by
    token, ``[N, rank + rot]``: the result is then the pair ``(rotated query parts, rows)``.  ``queries``
    (``[N, heads x (dim | rot)]``, rows may have a pitch): the queries lie there and ``proj`` holds ``[rank | rot]`` from
    column ``kv_col`` on (queries that come through a latent of their own are a later product than the keys' latent).
    ``halves``: the rotated lanes pair as ``(i, i + rot_dims / 2)`` instead of ``(2i, 2i + 1)``."""
    if queries is None:
        _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= heads * (dim + rot) + rank + rot, "latent_prepare: proj rows are too short")
    else:
        _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= kv_col + rank + rot, "latent_prepare: proj rows are too short")
        _need(queries.dim() == 2 and queries.stride(1) == 1 and queries.dtype == proj.dtype and queries.shape[0] == proj.shape[0]
              and queries.shape[1] >= heads * (dim + rot), "latent_prepare: the queries' rows are too short, or of another type")
    _need(plane.dtype == proj.dtype and plane.is_contiguous() and plane.dim() == 3 and plane.shape[2] == rank + rot, "latent_prepare: the plane must be [pages, page_size, rank + rot] of the rows' type")
    _need(weight.dtype == torch.float32 and weight.numel() == rank and freq.dtype == torch.float32 and freq.is_contiguous(), "latent_prepare: weight [rank] and freq are float32")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    rot_dims = 2 * freq.numel()
    q_rot = torch.empty((proj.shape[0], heads, rot), dtype=proj.dtype, device=proj.device)
    rows = torch.empty((proj.shape[0], rank + rot), dtype=proj.dtype, device=proj.device) if fresh else None
    code = _launch("llm_latent_prepare", _ptr(proj), _code(proj.dtype), proj.stride(0), _ptr(q_rot), _ptr(rows), _ptr(positions),
                   _ptr(slot_map), _ptr(plane), _ptr(weight), _ptr(freq), float(eps), proj.shape[0], heads, dim, rot, rank, rot_dims,
                   _ptr(queries), 0 if queries is None else queries.stride(0), int(kv_col), int(halves), _stream())
    _check(code, "latent_prepare")
    return (q_rot, rows) if fresh else q_rot


def unit_norm_kv_write(qkv: torch.Tensor, slot_map: torch.Tensor, pool: torch.Tensor, eps: float | None, heads: int, kv_heads: int,
                       key_dim: int, value_dim: int) -> None:
    """``qkv`` rows = ``[heads x key_dim | kv_heads x key_dim | kv_heads x value_dim]``.  With ``eps`` every query
    head (in place) and key head is divided by its root mean square ``sqrt(mean(x^2) + eps)``; keys and values are
    written to the row's slot of ``pool [pages, 2, kv_heads, page_size, D]`` (``D >= key_dim, value_dim``)."""
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= (heads + kv_heads) * key_dim + kv_heads * value_dim, "unit_norm_kv_write: qkv rows are too short")
    _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, kv_heads), "the pool plane does not match the heads")
    _need(pool.shape[4] >= max(key_dim, value_dim), "the pool's rows are shorter than a key or a value")
    _i32(slot_map, "slot_map")
    code = _launch("llm_unit_norm_kv_write", _ptr(qkv), _code(qkv.dtype), qkv.stride(0), _ptr(slot_map), _ptr(pool),
                   float(eps or 0.0), int(eps is not None), qkv.shape[0], heads, kv_heads, key_dim, value_dim, pool.shape[4],
                   pool.shape[3], _stream())
    _check(code, "unit_norm_kv_write")


def head_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """One product per head: ``x [N, heads, K]`` (any token and head strides) times ``w [heads, M, K]`` ->
    ``[N, heads, M]`` (a view whose strides the callers do not rely on).  float32 on the CUDA cores in true 32-bit;
    bfloat16 through the vendor's batched product, 32-bit accumulation."""
    _need(x.dim() == 3 and w.dim() == 3 and x.shape[1] == w.shape[0] and x.shape[2] == w.shape[2], f"head_linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype and x.stride(2) == 1 and w.is_contiguous(), "head_linear: operands of one type, unit inner strides")
    n, heads, k = x.shape
    m = w.shape[1]
    if x.dtype == torch.float32:
        out = torch.empty((n, heads, m), dtype=x.dtype, device=x.device)
        code = _launch("llm_gemm_simt_batched", _ptr(x), _ptr(w), _ptr(out), _F32, _F32, n, m, k, x.stride(0), k, heads * m,
                       heads, x.stride(1), m * k, m, _stream())
        _check(code, "head_linear (float32)")
        return out
    library()
    return torch.bmm(x.transpose(0, 1), w.transpose(1, 2)).transpose(0, 1)


def attention_rows(q0, q1, keys, k_strides, values, v_strides, value_dim: int, page_table, page_size: int, ctx, *, num_heads: int,
                   num_kv_heads: int, scale: float, window: int | None = None, slopes: torch.Tensor | None = None,
                   key_part: int = 0, keys1: int | None = None, k1_token: int = 0, fresh_d0: int = 0, want_stats: bool = False,
                   leave_parts: bool = False, sinks: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                   keep_first: int | None = None, chunk: int | None = None, softcap: float | None = None):
    """Attention in its general form: queries ``q0 [N, H, d0]`` and optionally ``q1 [N, H, d1]`` (lanes behind q0's),
    keys and values addressed by ``(page, head, token)`` strides in elements, an optional bias ``-slopes[h] * distance``.
    Returns ``[N, H, value_dim]``.

    ``key_part`` (bfloat16 on the tensor cores only): 1 = only the keys cached before this step; 2 = only the step's own
    tokens, whose keys and values lie token by token (``keys`` lanes ``[0, fresh_d0)`` per head, ``keys1`` the lanes
    behind them, one row a token for all heads).  With ``want_stats`` the result is ``(out, stats [N, H, 2])``: each row's
    maximum score and sum of exponentials (a row without keys: ``-inf, 0``, and an output that is not to be read), for :func:`merge_two_parts`.
    ``leave_parts``: where the keys are cut over several CTAs the partial results are not merged but returned as an
    :class:`AttentionParts`, for a kernel that merges them on its way (:func:`merge_project_gate`).
    ``sinks`` (float32 ``[H]``): every head's softmax has one more term ``exp(sinks[h])`` in its denominator, with no key and
    no value.  ``gate`` (float32 ``[N, >= H * value_dim]``, rows may have a pitch): the output is multiplied by its sigmoid.
    ``keep_first``: with a window, the keys at positions below it stay visible to every later query.  ``chunk``: a query sees
    only the keys of its own block of so many positions, counted from 0.  ``softcap``: a scaled score s becomes
    ``softcap * tanh(s / softcap)`` before the distance bias is taken off."""
    n, d0 = q0.shape[0], q0.shape[2]
    keep_first, chunk, softcap = int(keep_first or 0) if window else 0, int(chunk or 0), float(softcap or 0.0)
    _need(keep_first >= 0 and chunk >= 0 and softcap >= 0.0, "attention_rows: keep_first, chunk and softcap are not negative")
    if sinks is not None:
        _need(sinks.dtype == torch.float32 and sinks.numel() == num_heads and sinks.is_contiguous(), "sinks must be float32 [heads]")
    if gate is not None:
        _need(gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape[0] == n and gate.shape[1] >= num_heads * value_dim, "the gate must be float32 [N, heads * value_dim]")
        _need(not leave_parts, "a gate is applied where the output is written, not to partial results")
    gate_token = 0 if gate is None else gate.stride(0)
    d1 = 0 if q1 is None else q1.shape[2]
    _need(q0.stride(2) == 1 and (q1 is None or q1.stride(2) == 1), "attention_rows: queries need unit inner strides")
    _i32(page_table, "page_table")
    if slopes is not None:
        _need(slopes.dtype == torch.float32 and slopes.numel() == num_heads and slopes.is_contiguous(), "slopes must be float32 [heads]")
    out = torch.empty((n, num_heads, value_dim), dtype=q0.dtype, device=q0.device)
    if q0.dtype == torch.bfloat16 and not _FORCE_GENERIC_ATTENTION and d0 % 16 == 0 and d1 % 16 == 0 and value_dim % 16 == 0 and value_dim <= 256:
        # the tensor cores: 64 rows of (token, group member) a CTA; few CTAs and long contexts: the keys cut over several
        group = num_heads // num_kv_heads
        longest = getattr(ctx, "max_context_len", None) or int(ctx.context_lens.max())
        if window:
            longest = min(longest, window + keep_first + ctx.max_query_len)
        if chunk:
            longest = min(longest, chunk + ctx.max_query_len)
        ctas = -(-ctx.max_query_len * group // 64) * num_kv_heads * ctx.num_requests
        splits = max(1, min(-(-longest // 256), _sm_count() // ctas, 16, _SPLIT_SCRATCH_BYTES // (n * num_heads * value_dim * 4)))
        if key_part or want_stats:
            splits = 1
        stats = torch.empty((n, num_heads, 2), dtype=torch.float32, device=q0.device) if want_stats else None
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((n * num_heads * splits * value_dim,), dtype=torch.float32, device=q0.device)
            part_ml = torch.empty((n * num_heads * splits * 2,), dtype=torch.float32, device=q0.device)
        code = _launch(
            "llm_attention_rows_mma", _ptr(q0), q0.stride(0), q0.stride(1), d0, _ptr(q1), 0 if q1 is None else q1.stride(0),
            0 if q1 is None else q1.stride(1), d1, None if (leave_parts and splits > 1) else _ptr(out), out.stride(0), out.stride(1),
            keys, *k_strides, values, *v_strides,
            value_dim, _ptr(page_table), page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens), _ptr(ctx.context_lens),
            _ptr(slopes), n, ctx.num_requests, ctx.max_query_len, num_heads, num_kv_heads, page_size, int(window or 0), float(scale),
            splits, _ptr(part_o), _ptr(part_ml), int(key_part), keys1, int(k1_token), int(fresh_d0), _ptr(stats), _ptr(sinks), _ptr(gate),
            gate_token, keep_first, chunk, softcap, _stream(),
        )
        if code != 10002:
            _check(code, "attention_rows (tensor cores)")
            if leave_parts and splits > 1:
                return AttentionParts(part_o, part_ml, splits, n, num_heads, value_dim)
            add_launches(int(splits > 1))
            return (out, stats) if want_stats else out
        add_launches(-1)  # a layout the kernel does not take: the general one below
    _need(not key_part and not want_stats, "attention over a part of the keys runs on the tensor cores only (bfloat16, lanes in multiples of 16)")
    code = _launch(
        "llm_attention_rows", _ptr(q0), q0.stride(0), q0.stride(1), d0, _ptr(q1), 0 if q1 is None else q1.stride(0),
        0 if q1 is None else q1.stride(1), d1, _ptr(out), out.stride(0), out.stride(1), keys, *k_strides, values, *v_strides,
        value_dim, _code(q0.dtype), _ptr(page_table), page_table.shape[1], _ptr(ctx.token_request), _ptr(ctx.cu_tokens),
        _ptr(ctx.context_lens), _ptr(slopes), n, num_heads, num_kv_heads, page_size, int(window or 0), float(scale), _ptr(sinks),
        _ptr(gate), gate_token, keep_first, chunk, softcap, _stream(),
    )
    _check(code, "attention_rows")
    return out


class AttentionParts:
    """Partial results of attention whose keys were cut over ``splits`` CTAs: ``part_o [n * heads * splits * dv]``
    unnormalised outputs, ``part_ml [n * heads * splits * 2]`` each part's maximum and sum."""

    def __init__(self, part_o, part_ml, splits: int, n: int, heads: int, dv: int):
        self.part_o, self.part_ml, self.splits, self.n, self.heads, self.dv = part_o, part_ml, splits, n, heads, dv


def merge_project_gate(parts: AttentionParts, w: torch.Tensor, gate: torch.Tensor | None, per_head: bool = False) -> torch.Tensor:
    """``out[t, h * M + e] = sigmoid(gate[t, h * M + e]) * sum_r w[h, e, r] * merged[t, h, r]`` where ``merged`` is what
    :class:`AttentionParts` merge to: the merge, the product per head with ``w [heads, M, dv]`` (bfloat16) and the gate
    (None: none) in one kernel, for steps of few rows.  ``per_head``: one gate a head and token, ``gate [n, heads]``."""
    _need(w.dtype == torch.bfloat16 and w.is_contiguous() and w.dim() == 3 and w.shape[0] == parts.heads and w.shape[2] == parts.dv, "merge_project_gate: w [heads, M, dv] bfloat16")
    m = w.shape[1]
    if gate is not None:
        _need(gate.dtype == torch.bfloat16 and gate.stride(1) == 1 and tuple(gate.shape) == (parts.n, parts.heads if per_head else parts.heads * m),
              "merge_project_gate: gate [n, heads * M] (or [n, heads]) bfloat16")
    out = torch.empty((parts.n, parts.heads * m), dtype=torch.bfloat16, device=w.device)
    code = _launch("llm_merge_project_gate", _ptr(parts.part_o), _ptr(parts.part_ml), parts.splits, _ptr(w), _ptr(gate),
                   0 if gate is None else gate.stride(0), _ptr(out), parts.n, parts.heads, parts.dv, m, int(per_head), _stream())
    _check(code, "merge_project_gate")
    return out


def merge_two_parts(o1: torch.Tensor, stats1: torch.Tensor, o2: torch.Tensor, stats2: torch.Tensor) -> torch.Tensor:
    """Two parts of one softmax, each normalised by itself (``o [N, H, dv]`` bfloat16 with any token and head strides,
    ``stats [N, H, 2]``), joined: ``(w1 o1 + w2 o2) / (w1 + w2)`` with ``w = sum * exp(maximum - M)``."""
    _need(o1.shape == o2.shape and o1.dtype == o2.dtype == torch.bfloat16 and o1.stride(2) == 1 and o2.stride(2) == 1, "merge_two_parts: two bfloat16 [N, H, dv] outputs")
    n, heads, dv = o1.shape
    out = torch.empty((n, heads, dv), dtype=o1.dtype, device=o1.device)
    code = _launch("llm_merge_two_parts", _ptr(o1), o1.stride(0), o1.stride(1), _ptr(stats1), _ptr(o2), o2.stride(0), o2.stride(1),
                   _ptr(stats2), _ptr(out), out.stride(0), out.stride(1), n, heads, dv, _stream())
    _check(code, "merge_two_parts")
    return out


# from this many tokens of a request in a step on, latent attention expands the step's own keys and values per head
_LATENT_TWO_PART_MIN_TOKENS = 128


def latent_two_parts(ctx, dtype: torch.dtype, *lanes: int) -> bool:
    """Whether a step's latent attention runs in two parts (see parts/latent_attention.py): a bfloat16 step in which a
    request brings many tokens, with every run of lanes a multiple of 16."""
    return (dtype == torch.bfloat16 and not _FORCE_GENERIC_ATTENTION and ctx.max_query_len >= _LATENT_TWO_PART_MIN_TOKENS
            and all(x % 16 == 0 for x in lanes))


def latent_paged_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, plane: torch.Tensor, page_table: torch.Tensor, ctx, *,
                           rank: int, scale: float, window: int | None = None, cached_only: bool = False, leave_parts: bool = False):
    """Attention of every new token over its request's cached latents.  A cached row ``[rank | rot]`` is the key of
    every head (against the query ``[q_lat | q_rot]``) and, in its first ``rank`` lanes, the value.
    ``plane [pages, page_size, rank + rot]``; returns ``[N, H, rank]``.  ``cached_only``: only the rows cached before
    this step are seen, and the result is ``(out, stats)`` for :func:`merge_two_parts`."""
    _need(plane.dtype == q_lat.dtype and plane.is_contiguous() and plane.dim() == 3, "the plane must be contiguous [pages, page_size, width] of the query type")
    page_size, width = plane.shape[1], plane.shape[2]
    _need(q_lat.shape[2] == rank and q_lat.shape[2] + q_rot.shape[2] == width, "the queries do not match the cached rows")
    strides = (page_size * width, 0, width)
    return attention_rows(q_lat, q_rot, _ptr(plane), strides, _ptr(plane), strides, rank, page_table, page_size, ctx,
                          num_heads=q_lat.shape[1], num_kv_heads=1, scale=scale, window=window,
                          key_part=1 if cached_only else 0, want_stats=cached_only, leave_parts=leave_parts and not cached_only)


def fresh_latent_attention(q_plain: torch.Tensor, q_rot: torch.Tensor, kv: torch.Tensor, fresh: torch.Tensor, page_table: torch.Tensor,
                           ctx, *, dim: int, value_dim: int, rank: int, scale: float, window: int | None = None, want_stats: bool = True):
    """Attention of every new token over the step's own tokens of its request, with keys and values per head:
    ``kv [N, H * dim | H * value_dim]`` (the latents' products with the two up matrices), the rotated shared key part in
    ``fresh[:, rank:]``.  Returns ``(out [N, H, value_dim], stats)`` for :func:`merge_two_parts`, or ``out`` alone
    without ``want_stats``."""
    n, heads = q_plain.shape[0], q_plain.shape[1]
    rot = fresh.shape[1] - rank
    _need(kv.is_contiguous() and fresh.is_contiguous() and kv.shape[1] == heads * (dim + value_dim), "fresh_latent_attention: kv [N, H dim | H vdim]")
    element = kv.element_size()
    return attention_rows(q_plain, q_rot, kv.data_ptr(), (0, dim, kv.stride(0)), kv.data_ptr() + heads * dim * element,
                          (0, value_dim, kv.stride(0)), value_dim, page_table, 1, ctx, num_heads=heads, num_kv_heads=heads,
                          scale=scale, window=window, key_part=2, keys1=fresh.data_ptr() + rank * element, k1_token=rank + rot,
                          fresh_d0=dim, want_stats=want_stats)


def biased_paged_attention(qkv: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                           key_dim: int, value_dim: int, scale: float, window: int | None = None,
                           slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped-query attention whose keys and values may differ in size and whose scores may lose
    ``slopes[h] * distance``.  ``qkv`` rows start with the query heads (``key_dim`` each); keys and values are in
    ``pool [pages, 2, kv_heads, page_size, D]``.  Returns ``[N, num_heads * value_dim]``."""
    _need(qkv.stride(1) == 1 and qkv.shape[1] >= num_heads * key_dim, "qkv rows must start with the query heads")
    _need(pool.dtype == qkv.dtype and pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, num_kv_heads), "the pool plane does not match the heads")
    page_size, row = pool.shape[3], pool.shape[4]
    _need(row >= max(key_dim, value_dim), "the pool's rows are shorter than a key or a value")
    q = qkv.as_strided((qkv.shape[0], num_heads, key_dim), (qkv.stride(0), key_dim, 1), qkv.storage_offset())
    head, page = page_size * row, 2 * num_kv_heads * page_size * row
    values = pool.data_ptr() + num_kv_heads * head * pool.element_size()
    out = attention_rows(q, None, _ptr(pool), (page, head, row), values, (page, head, row), value_dim, page_table, page_size, ctx,
                         num_heads=num_heads, num_kv_heads=num_kv_heads, scale=scale, window=window, slopes=slopes)
    return out.view(qkv.shape[0], num_heads * value_dim)


def paged_softmax_attention(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                            key_dim: int, value_dim: int, scale: float, window: int | None = None, sinks: torch.Tensor | None = None,
                            gate: torch.Tensor | None = None, keep_first: int | None = None, chunk: int | None = None,
                            softcap: float | None = None, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped-query softmax attention of prepared queries ``q [N, num_heads * key_dim]`` over keys and values in
    ``pool [pages, 2, kv_heads, page_size, D]`` (``D >= key_dim, value_dim``), with an optional sink per head and an
    optional sigmoid gate on the output, a window that may keep the first keys, blocks of positions, a cap on the scores and a
    distance bias per head (see :func:`attention_rows`).  Returns ``[N, num_heads * value_dim]``."""
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] == num_heads * key_dim, "paged_softmax_attention: q [N, heads * key_dim]")
    _need(pool.dtype == q.dtype and pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, num_kv_heads), "the pool plane does not match the heads")
    page_size, row = pool.shape[3], pool.shape[4]
    _need(row >= max(key_dim, value_dim), "the pool's rows are shorter than a key or a value")
    q3 = q.as_strided((q.shape[0], num_heads, key_dim), (q.stride(0), key_dim, 1), q.storage_offset())
    head, page = page_size * row, 2 * num_kv_heads * page_size * row
    values = pool.data_ptr() + num_kv_heads * head * pool.element_size()
    out = attention_rows(q3, None, _ptr(pool), (page, head, row), values, (page, head, row), value_dim, page_table, page_size, ctx,
                         num_heads=num_heads, num_kv_heads=num_kv_heads, scale=scale, window=window, sinks=sinks, gate=gate,
                         keep_first=keep_first, chunk=chunk, softcap=softcap, slopes=slopes)
    return out.view(q.shape[0], num_heads * value_dim)


def head_prepare(proj: torch.Tensor, positions: torch.Tensor | None, *, heads: int, kv_heads: int, dim: int, value_dim: int = 0,
                 bias: torch.Tensor | None = None, q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None,
                 eps: float = 0.0, freq: torch.Tensor | None = None, warm: tuple[float, int] | None = None,
                 values_are_keys: bool = False, pool: torch.Tensor | None = None, slot_map: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None, interleaved: bool = False, values_out: torch.Tensor | None = None,
                 values_first: torch.Tensor | None = None, values_lambda: float = 0.0) -> torch.Tensor:
    """From a token's stacked projections ``proj`` rows ``[heads x dim | kv_heads x dim | kv_heads x value_dim]`` to
    queries, keys and values, in this order: ``bias`` (float32, laid out like the row) is added; with ``q_weight`` /
    ``k_weight`` (float32 ``[dim]``) every head is RMS-normed over its lanes (``eps`` inside the root) and weighted; with
    ``freq`` (float32 ``[rot / 2]``) lanes ``i`` and ``i + rot/2`` of every head turn by ``position * freq[i]``; with
    ``warm = (coef, every)`` queries are multiplied by ``1 + coef * ln(floor((position + 1) / every) + 1)``.  Keys and values
    go to the tokens' slots of ``pool [pages, 2, kv_heads, page_size, D]``; with ``values_are_keys`` there are no value
    columns and a key head's value is that head with its bias, before norm and rotation.  ``kv_heads = 0``: queries only.
    ``interleaved``: the rotated lanes pair as ``(2i, 2i + 1)``.  ``values_out`` (float32 ``[N, kv_heads * value_dim]``)
    takes the values as projected, bias included; with ``values_first`` (the same shape: what an earlier layer kept for
    these tokens) the values become ``(1 - values_lambda) v + values_lambda values_first`` on their way to the pool.
    Returns the queries ``[N, heads * dim]`` in ``out_dtype`` (default: the pool's type)."""
    cols = (heads + kv_heads) * dim + (0 if values_are_keys else kv_heads * value_dim)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= cols, "head_prepare: proj rows are too short")
    n = proj.shape[0]
    rot = 0
    if freq is not None:
        _need(freq.dtype == torch.float32 and freq.is_contiguous(), "head_prepare: freq is float32")
        rot = 2 * freq.numel()
    if rot or warm:
        _i32(positions, "positions")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == cols, "head_prepare: the bias is float32, laid out like the row")
    normed = q_weight is not None
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == dim), "head_prepare: norm weights are float32 [dim]")
    if kv_heads:
        _need(pool is not None and pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, kv_heads), "the pool plane does not match the heads")
        _need(not normed or k_weight is not None, "head_prepare: normed keys need a weight")
        _i32(slot_map, "slot_map")
        out_dtype = pool.dtype
    out_dtype = out_dtype or proj.dtype
    for t in (values_out, values_first):
        _need(t is None or (kv_heads and not values_are_keys and t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == (n, kv_heads * value_dim)),
              "head_prepare: the values kept for, or taken from, another layer are float32 [N, kv_heads * value_dim]")
    q = torch.empty((n, heads * dim), dtype=out_dtype, device=proj.device)
    coef, every = (float(warm[0]), int(warm[1])) if warm else (0.0, 0)
    code = _launch(
        "llm_head_prepare", _ptr(proj), _code(proj.dtype), proj.stride(0), _ptr(bias), _ptr(q), q.stride(0), _ptr(pool) if kv_heads else None,
        _code(out_dtype), _ptr(slot_map) if kv_heads else None, pool.shape[3] if kv_heads else 1, pool.shape[4] if kv_heads else dim,
        _ptr(q_weight), _ptr(k_weight), float(eps), int(normed), _ptr(freq), rot, _ptr(positions) if (rot or warm) else None, coef, every,
        n, heads, kv_heads, dim, value_dim, int(values_are_keys), int(interleaved), _ptr(values_out), _ptr(values_first), float(values_lambda),
        _stream(),
    )
    _check(code, "head_prepare")
    return q


def hyper_mix_norm(streams: torch.Tensor, update: "StreamUpdate | None", read_in: torch.Tensor | None, weight: torch.Tensor, eps: float,
                   rows: torch.Tensor | None = None, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """One pass over the copies ``streams [S, N, W]`` (float32) of a residual stream between two parts: with ``update`` the
    copies take up what the part in front returned, ``x_t <- sum_s mix[s, t] x_s + take[t] * result`` (in place); then
    ``u = sum_t read_in[t] x_t`` (``read_in`` None: the plain sum) and the result is ``u * rsqrt(mean(u^2) + eps) * weight``
    in ``out_dtype``.  With ``rows`` (int32) only those rows are produced and the copies are left as they were."""
    _need(streams.dtype == torch.float32 and streams.dim() == 3 and streams.is_contiguous(), "hyper_mix_norm: the copies are contiguous float32 [S, N, W]")
    S, n, w = streams.shape
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == w, "hyper_mix_norm: the norm weight is float32 [W]")
    ys, fs = ([], [])
    if update is not None:
        ys, fs = update.results()
        _need(1 <= len(ys) <= 4, "hyper_mix_norm: a part's result is a weighted sum of one to four tensors")
        for y in ys:
            _need(y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (n, w), "hyper_mix_norm: results are contiguous float32 [N, W]")
        for t, size in ((update.mix, S * S), (update.take, S)):
            _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == size, "hyper_mix_norm: mix [S, S] and take [S] are float32")
    if read_in is not None:
        _need(read_in.dtype == torch.float32 and read_in.is_contiguous() and read_in.numel() == S, "hyper_mix_norm: read_in is float32 [S]")
    if rows is not None:
        _i32(rows, "rows")
    n_out = n if rows is None else rows.numel()
    out = torch.empty((n_out, w), dtype=out_dtype, device=streams.device)
    yp = [_ptr(ys[i]) if i < len(ys) else None for i in range(4)]
    fp = [float(fs[i]) if i < len(fs) else 0.0 for i in range(4)]
    code = _launch("llm_hyper_mix_norm", _ptr(streams), *yp, *fp, len(ys), _ptr(update.mix) if update is not None else None,
                   _ptr(update.take) if update is not None else None, _ptr(read_in), _ptr(weight), float(eps), _ptr(rows), _ptr(out),
                   _code(out_dtype), n_out, S, n, w, _stream())
    _check(code, "hyper_mix_norm")
    return out


def linear32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T`` for an input that stays 32-bit whatever the weights' type: true 32-bit multiply-adds on
    the CUDA cores, float32 out (a small product on the way into a recurrence)."""
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == torch.float32, f"linear32: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match, or x is not float32")
    _need(x.stride(1) == 1 and w.is_contiguous(), "linear32: operands must have unit inner stride")
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    code = _launch("llm_gemm_simt", _ptr(x), _F32, _ptr(w), _code(w.dtype), _ptr(out), _F32, m, n, k, x.stride(0), k, n, _stream())
    _check(code, "linear32")
    return out


def gated_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: torch.Tensor | None, inv_tau: float,
               q_scale: float, states: torch.Tensor, state_slots: torch.Tensor, cu_tokens: torch.Tensor, num_requests: int, heads: int,
               dim: int, value_dim: int, max_query_len: int = 0) -> torch.Tensor:
    """``S = diag(alpha_t) S + k_t v_t^T``, ``o_t = S^T (q_scale * q_t)`` per head over every request's new tokens, with a
    decay per key channel that the token chooses: ``alpha_t = sigmoid(z_t + z_bias) ^ inv_tau``.  From and to
    ``states[state_slots[r]]`` (``[slots, heads, dim, value_dim]`` float32).  ``q, k, z [N, heads * dim]`` float32 and
    ``v [N, heads * value_dim]`` (views with a row pitch will do).  Returns ``o [N, heads, value_dim]`` float32.  Long
    requests are shared out over several CTAs in stretches, as in :func:`retention_scan` (the same kernel walks both)."""
    for t in (q, k, z):
        _need(t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[1] == heads * dim, "gated_scan: q, k and the decays' logits are float32 [N, heads * dim]")
    _need(v.stride(1) == 1 and v.shape[1] == heads * value_dim, "gated_scan: v [N, heads * value_dim]")
    _need(states.dtype == torch.float32 and states.is_contiguous() and tuple(states.shape[1:]) == (heads, dim, value_dim), "gated_scan: states [slots, heads, dim, value_dim] float32")
    _need(z_bias is None or (z_bias.dtype == torch.float32 and z_bias.is_contiguous() and z_bias.numel() == heads * dim), "gated_scan: the bias is float32 [heads * dim]")
    _i32(state_slots, "state_slots")
    _i32(cu_tokens, "cu_tokens")
    out = torch.empty((q.shape[0], heads, value_dim), dtype=torch.float32, device=q.device)
    few = 0 < int(max_query_len) <= 16
    stretches = _scan_stretches(few, dim, value_dim, heads, int(num_requests), int(max_query_len))
    scratch = None
    if stretches > 1:  # the stretches' end states, start states and products of decays
        scratch = torch.empty((int(num_requests) * stretches * heads * (2 * dim * value_dim + dim),), dtype=torch.float32, device=q.device)
    code = _launch("llm_gated_scan", _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), _code(v.dtype), v.stride(0), _ptr(z), z.stride(0),
                   _ptr(z_bias), float(inv_tau), float(q_scale), _ptr(states), _ptr(state_slots), _ptr(cu_tokens), _ptr(out), int(num_requests),
                   heads, dim, value_dim, stretches, _ptr(scratch), int(few), _stream())
    add_launches(2 * int(stretches > 1))
    _check(code, "gated_scan")
    return out


def expert_gated_act(x: torch.Tensor, experts: int, ff: int, shared_ff: int, limit: float, shared_limit: float, slope: float, *,
                     weights: torch.Tensor | None = None, ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                     up_shift: float = 1.0) -> torch.Tensor:
    """The activation of gated experts whose products are bounded, times each token's weight of the expert:
    ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``y = g * sigmoid(slope * g) * (u + up_shift) * weight``
    (infinite limits, slope 1 and shift 0: ``silu(gate) * up * weight``).
    ``x [N, experts * 2 ff + 2 shared_ff]``: per expert its gate columns, then its up columns; a shared expert's behind them
    (``shared_limit``).  The weight is ``weights[t, e]`` (float32 ``[N, experts (+ 1)]``) or, from ``ids [N]`` and
    ``table [vocab, top]`` (int32), ``1 / top`` for the experts that the table lists for the token's id, 0 for the others and
    1 for the shared one.  Returns ``[N, experts * ff + shared_ff]``."""
    _need(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= 2 * (experts * ff + shared_ff), "expert_gated_act: x rows hold every expert's gate and up columns")
    top = vocab = ldw = 0
    if weights is not None:
        _need(weights.dtype == torch.float32 and weights.stride(1) == 1 and weights.shape[0] == x.shape[0] and weights.shape[1] >= experts + int(shared_ff > 0), "expert_gated_act: weights are float32 [N, experts (+ 1)]")
        ldw = weights.stride(0)
    else:
        _i32(ids, "ids")
        _need(table is not None and table.dtype == torch.int32 and table.is_contiguous() and table.dim() == 2 and ids.numel() == x.shape[0], "expert_gated_act: table is int32 [vocab, top]")
        vocab, top = table.shape
    out = torch.empty((x.shape[0], experts * ff + shared_ff), dtype=x.dtype, device=x.device)
    code = _launch("llm_expert_gated_act", _ptr(x), x.stride(0), _ptr(out), out.stride(0), _code(x.dtype), _ptr(weights), ldw, _ptr(ids),
                   _ptr(table), top, vocab, x.shape[0], experts, ff, shared_ff, float(limit), float(shared_limit), float(slope), float(up_shift), _stream())
    _check(code, "expert_gated_act")
    return out


# ------------------------------------------------------------------------------------------------
# Operations of layers whose attention weighs keys by a sigmoid and mixes the heads' weights, that keep a decaying
# matrix of state per head, that route tokens to a few of many small feed-forward layers, or that run mixers side by
# side (csrc/sigmoid_attention.cu, retention.cu, routing.cu).
_SIGMOID_SPLIT_KEYS = 128  # a stretch of keys that one CTA sums up when a context is shared out
_SIGMOID_SPLIT_MAX_TOKENS = 64  # steps of more tokens have CTAs enough without cutting the keys
_SIGMOID_SHARES = 16  # the tensor-core kernel's CTAs per tile of tokens: stretch s of the keys goes to share s % 16


def qk_prepare(proj: torch.Tensor, positions: torch.Tensor | None, *, heads: int, kv_heads: int, dim: int, value_dim: int = 0,
               freq: torch.Tensor | None = None, q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None,
               eps: float = 0.0, k_scale: float = 1.0, pool: torch.Tensor | None = None, slot_map: torch.Tensor | None = None,
               out_dtype: torch.dtype | None = None):
    """From a token's stacked projections ``proj`` rows ``[heads x dim | kv_heads x dim | kv_heads x value_dim | ...]``
    to queries and keys: with ``q_weight`` / ``k_weight`` (float32, the whole projection's size) the query projection and
    the key projection are each RMS-normed as one vector (``eps`` inside the root) and weighted; with ``freq``
    (float32 ``[rot / 2]``) lanes ``i`` and ``i + rot/2`` of every head turn by ``position * freq[i]`` (32-bit angles);
    keys are multiplied by ``k_scale``.  With ``pool [pages, 2, kv_heads, page_size, D]`` keys and values go to the
    tokens' slots and the queries ``[N, heads * dim]`` (``out_dtype``, default the pool's type) are returned; without,
    ``(queries, keys [N, kv_heads * dim])`` in ``out_dtype`` are."""
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= (heads + kv_heads) * dim + (kv_heads * value_dim if pool is not None else 0), "qk_prepare: proj rows are too short")
    n = proj.shape[0]
    rot = 0
    if freq is not None:
        _need(freq.dtype == torch.float32 and freq.is_contiguous(), "qk_prepare: freq is float32")
        _i32(positions, "positions")
        rot = 2 * freq.numel()
    for w, size in ((q_weight, heads * dim), (k_weight, kv_heads * dim)):
        _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == size), "qk_prepare: norm weights are float32 of the projection's size")
    if pool is not None:
        _need(pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, kv_heads), "the pool plane does not match the heads")
        _i32(slot_map, "slot_map")
        out_dtype = pool.dtype
    out_dtype = out_dtype or proj.dtype
    q = torch.empty((n, heads * dim), dtype=out_dtype, device=proj.device)
    k = None if pool is not None else torch.empty((n, kv_heads * dim), dtype=out_dtype, device=proj.device)
    code = _launch(
        "llm_qk_prepare", _ptr(proj), _code(proj.dtype), proj.stride(0), _ptr(q), _code(out_dtype), q.stride(0), _ptr(k),
        0 if k is None else k.stride(0), _ptr(pool), _code(out_dtype), _ptr(slot_map), 0 if pool is None else pool.shape[3],
        0 if pool is None else pool.shape[4], _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(freq), rot, _ptr(positions),
        float(k_scale), n, heads, kv_heads, dim, value_dim, _stream(),
    )
    _check(code, "qk_prepare")
    return q if pool is not None else (q, k)


def sigmoid_attention(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                      key_dim: int, value_dim: int, scale: float, softcap: float | None = None, head_bias: torch.Tensor | None = None,
                      head_mix: torch.Tensor | None = None, window: int | None = None) -> torch.Tensor:
    """Attention whose weights are not normalised over keys: key j (``j <= i``, within ``window`` if there is one) gets
    ``sigmoid(cap(scale * q_g . k_j) + head_bias[g])`` with ``cap(s) = softcap * tanh(s / softcap)``, the heads' weights
    are mixed (``w_h = sum_g head_mix[h, g] p_g``) and head h sums up the values of its own key/value head with them.
    ``q [N, heads * key_dim]``; keys and values in ``pool [pages, 2, kv_heads, page_size, D]``.  Returns
    ``[N, heads * value_dim]``.  A step of few tokens shares long contexts out over several CTAs in stretches of a fixed
    number of keys and adds the partial sums in order."""
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] == num_heads * key_dim, "sigmoid_attention: q [N, heads * key_dim]")
    _need(pool.dtype == q.dtype and pool.is_contiguous() and pool.dim() == 5 and tuple(pool.shape[1:3]) == (2, num_kv_heads), "the pool plane does not match the heads")
    _i32(page_table, "page_table")
    for name, t, size in (("head_bias", head_bias, num_heads), ("head_mix", head_mix, num_heads * num_heads)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == size), f"sigmoid_attention: {name} is float32 of the heads' size")
    n = q.shape[0]
    out = torch.empty((n, num_heads * value_dim), dtype=q.dtype, device=q.device)
    longest = getattr(ctx, "max_context_len", None) or int(ctx.context_lens.max())
    if window:
        longest = min(longest, window + ctx.max_query_len)
    split_keys = max(_SIGMOID_SPLIT_KEYS, -(-longest // (1024 * 32)) * 32)  # at most 1,024 stretches, of whole chunks of 32 keys
    splits = 1 if n > _SIGMOID_SPLIT_MAX_TOKENS else max(1, -(-longest // split_keys))
    parts = torch.empty((splits, n, num_heads * value_dim), dtype=torch.float32, device=q.device) if splits > 1 else None
    if q.dtype == torch.bfloat16 and not _FORCE_GENERIC_ATTENTION:
        # the tensor cores: tiles of 16 tokens of one request
        cu = getattr(ctx, "host_cu_tokens", None) or ctx.cu_tokens.tolist()
        tiles = sum(-(-(b - a) // 16) for a, b in zip(cu[:-1], cu[1:]))
        code = _launch(
            "llm_sigmoid_attention_mma", _ptr(q), q.stride(0), _ptr(pool), _ptr(page_table), page_table.shape[1], _ptr(ctx.positions),
            _ptr(ctx.cu_tokens), _ptr(head_bias), _ptr(head_mix), _ptr(out), _ptr(parts), tiles, n, len(cu) - 1, num_heads, num_kv_heads,
            key_dim, value_dim, pool.shape[4], pool.shape[3], float(scale), float(softcap or 0.0), int(window or 0), split_keys, splits,
            _stream(),
        )
        if code != 10002:
            _check(code, "sigmoid_attention (tensor cores)")
            if splits > 1:
                _check(_launch("llm_sigmoid_sum_parts", _ptr(parts), _ptr(out), _code(out.dtype), _ptr(ctx.positions), n,
                               num_heads * value_dim, split_keys, int(window or 0), min(splits, _SIGMOID_SHARES), _stream()),
                       "sigmoid_attention (sum of the stretches)")
            return out
        add_launches(-1)  # sizes the kernel does not take: the general one below
    code = _launch(
        "llm_sigmoid_attention", _ptr(q), _code(q.dtype), q.stride(0), _ptr(pool), _code(pool.dtype), _ptr(page_table),
        page_table.shape[1], _ptr(ctx.positions), _ptr(ctx.token_request), _ptr(head_bias), _ptr(head_mix), _ptr(out),
        _code(out.dtype), _ptr(parts), n, num_heads, num_kv_heads, key_dim, value_dim, pool.shape[4], pool.shape[3], float(scale),
        float(softcap or 0.0), int(window or 0), split_keys, splits, _stream(),
    )
    _check(code, "sigmoid_attention")
    add_launches(int(splits > 1))
    return out


_RETENTION_MIN_STRETCH = 64  # tokens a stretch of a long request has at least


def _scan_stretches(few: bool, dim: int, value_dim: int, heads: int, requests: int, max_query_len: int) -> int:
    """Into how many stretches the scans (csrc/retention.cu) cut a long request, so that the GPU has CTAs enough."""
    cols = 16 if few else 64 if dim <= 64 else 32 if dim <= 128 else 16  # columns of the state that one CTA owns
    ctas = -(-value_dim // cols) * heads * requests
    return max(1, min(8, max_query_len // _RETENTION_MIN_STRETCH, -(-4 * _sm_count() // ctas), 65535 // max(1, requests)))


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, states: torch.Tensor,
                   state_slots: torch.Tensor, cu_tokens: torch.Tensor, num_requests: int, heads: int, dim: int, value_dim: int,
                   max_query_len: int = 0) -> torch.Tensor:
    """``S = decay[h] * S + k_t v_t^T``, ``o_t = S^T q_t`` per head over every request's new tokens
    ``cu_tokens[r]:cu_tokens[r+1]``, from and to ``states[state_slots[r]]`` (``[slots, heads, dim, value_dim]``
    float32).  ``q, k [N, heads * dim]`` float32, ``v [N, heads * value_dim]`` (a view with a row pitch will do).
    Returns ``o [N, heads, value_dim]`` float32.  ``max_query_len``: the most tokens a request brings; long requests are
    shared out over several CTAs in stretches (each walked from a zero state, the start states found by a short pass
    over the stretches' end states, the missing term added in a third launch)."""
    _need(q.dtype == torch.float32 and k.dtype == torch.float32 and q.stride(1) == 1 and k.stride(1) == 1, "retention_scan: queries and keys are float32")
    _need(v.stride(1) == 1 and v.shape[1] == heads * value_dim, "retention_scan: v [N, heads * value_dim]")
    _need(states.dtype == torch.float32 and states.is_contiguous() and tuple(states.shape[1:]) == (heads, dim, value_dim), "retention_scan: states [slots, heads, dim, value_dim] float32")
    _need(decay.dtype == torch.float32 and decay.is_contiguous() and decay.numel() == heads, "retention_scan: decay is float32 [heads]")
    _i32(state_slots, "state_slots")
    _i32(cu_tokens, "cu_tokens")
    out = torch.empty((q.shape[0], heads, value_dim), dtype=torch.float32, device=q.device)
    few = 0 < int(max_query_len) <= 16  # a decode step, or portions of a few tokens
    stretches = _scan_stretches(few, dim, value_dim, heads, int(num_requests), int(max_query_len))
    scratch = None
    if stretches > 1:
        scratch = torch.empty((2, int(num_requests) * stretches, heads, dim, value_dim), dtype=torch.float32, device=q.device)
    code = _launch("llm_retention_scan", _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), _code(v.dtype), v.stride(0), _ptr(decay),
                   _ptr(states), _ptr(state_slots), _ptr(cu_tokens), _ptr(out), int(num_requests), heads, dim, value_dim, stretches,
                   _ptr(scratch), int(few), _stream())
    _check(code, "retention_scan")
    add_launches(2 * int(stretches > 1))
    return out


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor | None, eps: float | None, kind: str = "silu",
                   out_dtype: torch.dtype = torch.float32, weight: torch.Tensor | None = None) -> torch.Tensor:
    """``o [N, heads, W]`` (float32): every head divided by its root mean square ``sqrt(mean(o^2) + eps)`` (``eps`` None:
    not) and multiplied by ``weight`` (float32 ``[W]``, the same for every head; None: not), times ``kind`` (``silu`` or
    ``sigmoid``) of ``gate [N, heads * W]`` (None: no gate) -> ``[N, heads * W]``."""
    _need(weight is None or (weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == o.shape[2]), "head_norm_gate: the weight is float32 [W]")
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.dim() == 3, "head_norm_gate: o is contiguous float32 [N, heads, W]")
    n, heads, w = o.shape
    if gate is not None:
        _need(gate.stride(1) == 1 and gate.shape[1] == heads * w and kind in _GATE_KINDS, "head_norm_gate: gate [N, heads * W]")
    out = torch.empty((n, heads * w), dtype=out_dtype, device=o.device)
    code = _launch("llm_head_norm_gate", _ptr(o), _ptr(gate), _code(gate.dtype) if gate is not None else _code(out_dtype),
                   0 if gate is None else gate.stride(0), _ptr(out), _code(out_dtype), n, heads, w,
                   -1.0 if eps is None else float(eps), _GATE_KINDS[kind] if gate is not None else -1, _ptr(weight), _stream())
    _check(code, "head_norm_gate")
    return out


def route_topk(z: torch.Tensor, correction: torch.Tensor | None, experts: int, top: int, scale: float = 1.0,
               renormalize: bool = False, shared_gate: bool = False) -> torch.Tensor:
    """Router weights of every token as a dense matrix.  ``z [N, >= experts (+ 1)]`` float32 logits; ``s = softmax`` over
    the first ``experts``; the ``top`` experts with the largest ``s + correction`` are chosen (the lowest index among
    equals) and get ``scale * s`` (over the chosen ones' sum with ``renormalize``), the others 0.  With ``shared_gate``
    a last column holds ``sigmoid(z[:, experts])``.  Returns ``[N, experts (+ 1)]`` float32."""
    _need(z.dtype == torch.float32 and z.dim() == 2 and z.stride(1) == 1, "route_topk: logits are float32")
    _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == experts), "route_topk: correction is float32 [experts]")
    out = torch.empty((z.shape[0], experts + int(shared_gate)), dtype=torch.float32, device=z.device)
    code = _launch("llm_route_topk", _ptr(z), z.stride(0), _ptr(correction), _ptr(out), z.shape[0], experts, top, float(scale),
                   int(renormalize), int(shared_gate), _stream())
    _check(code, "route_topk")
    return out


def route(x: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor | None, experts: int, top: int, scale: float = 1.0,
          renormalize: bool = False, shared_gate: bool = False, bias: torch.Tensor | None = None, shared_one: bool = False) -> torch.Tensor:
    """The router's 32-bit product and :func:`route_topk` in one kernel: ``x [N, K]`` (float32 or bfloat16, read as 32-bit),
    ``w_router [experts (+ 1), K]`` float32 (its last row the shared expert's gate with ``shared_gate``).  A token's sums
    are added in an order of their own, whatever else the step holds.  ``bias`` (float32 ``[experts]``) is added to the
    logits before anything else.  ``shared_one``: a last column of ones (a shared expert without a gate; the router has no
    row for it).  With ``renormalize`` and no correction the weights are the softmax over the chosen logits alone.
    Returns ``[N, experts (+ 1)]`` float32."""
    _need(not (shared_gate and shared_one), "route: a shared expert has a gate or the weight one, not both")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == experts), "route: bias is float32 [experts]")
    rows = experts + int(shared_gate)
    _need(x.dim() == 2 and x.stride(1) == 1 and w_router.dtype == torch.float32 and w_router.is_contiguous()
          and tuple(w_router.shape) == (rows, x.shape[1]), "route: x [N, K], w_router float32 [experts (+ 1), K]")
    _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == experts), "route: correction is float32 [experts]")
    out = torch.empty((x.shape[0], rows + int(shared_one)), dtype=torch.float32, device=x.device)
    code = _launch("llm_router", _ptr(x), _code(x.dtype), x.stride(0), _ptr(w_router), _ptr(correction), _ptr(out), x.shape[0], x.shape[1],
                   experts, top, float(scale), int(renormalize), 2 if shared_one else int(shared_gate), _ptr(bias), _stream())
    _check(code, "route")
    return out


def expert_act_scale(x: torch.Tensor, weights: torch.Tensor, experts: int, ff: int, activation: str) -> torch.Tensor:
    """``act(x[t, j]) * weights[t, j // ff]`` for the first ``experts * ff`` columns, ``* weights[t, experts]`` for
    the columns behind them (a shared expert's); ``x [N, C]``, ``weights`` float32."""
    _need(activation in _UNARY_KINDS and x.dim() == 2 and x.stride(1) == 1, f"expert_act_scale: activation {activation!r}")
    _need(weights.dtype == torch.float32 and weights.stride(1) == 1 and weights.shape[0] == x.shape[0], "expert_act_scale: weights are float32 [N, blocks]")
    _need(weights.shape[1] >= experts + int(x.shape[1] > experts * ff), "expert_act_scale: a weight per block of columns")
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    code = _launch("llm_expert_act_scale", _ptr(x), x.stride(0), _ptr(weights), weights.stride(0), _ptr(out), out.stride(0),
                   _code(x.dtype), x.shape[0], x.shape[1], experts, ff, _UNARY_KINDS[activation], _stream())
    _check(code, "expert_act_scale")
    return out


def branch_norm_sum(branches: list[torch.Tensor], weights: list[torch.Tensor], eps: float, factor: float) -> torch.Tensor:
    """``factor * sum_b rmsnorm(branches[b]) * weights[b]`` row by row: float32 ``[N, C]`` tensors (up to four), each
    divided by its own root mean square (``eps`` inside the root)."""
    _need(1 <= len(branches) <= 4 and len(weights) == len(branches), "branch_norm_sum: one to four branches, a weight each")
    n, c = branches[0].shape
    for x, w in zip(branches, weights):
        _need(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (n, c), "branch_norm_sum: branches are contiguous float32 of one shape")
        _need(w.dtype == torch.float32 and w.is_contiguous() and w.numel() == c, "branch_norm_sum: weights are float32 of the row size")
    out = torch.empty((n, c), dtype=torch.float32, device=branches[0].device)
    ptrs = []
    for i in range(4):
        ptrs += [_ptr(branches[i]), _ptr(weights[i])] if i < len(branches) else [None, None]
    code = _launch("llm_branch_norm_sum", *ptrs, len(branches), _ptr(out), n, c, float(eps), float(factor), _stream())
    _check(code, "branch_norm_sum")
    return out


def branch_sum_rmsnorm(pending: BranchSum, resid: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor | None:
    """``resid += pending`` (see :class:`BranchSum`) in place, then ``resid * rsqrt(mean(resid^2) + eps) * weight`` in
    ``out_dtype``, as one kernel.  None (nothing changed) where the rows do not fit its shared memory."""
    n, c = resid.shape
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == c, "branch_sum_rmsnorm: a float32 stream and norm weight")
    for x, w in zip(pending.branches, pending.weights):
        _need(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (n, c) and w.dtype == torch.float32 and w.numel() == c, "branch_sum_rmsnorm: branches are contiguous float32 of the stream's shape")
    out = torch.empty((n, c), dtype=out_dtype, device=resid.device)
    ptrs = []
    for i in range(4):
        ptrs += [_ptr(pending.branches[i]), _ptr(pending.weights[i])] if i < len(pending.branches) else [None, None]
    code = _launch("llm_branch_sum_norm", *ptrs, len(pending.branches), _ptr(resid), _ptr(weight), _ptr(out), _code(out_dtype), n, c,
                   pending.eps, pending.factor, float(eps), _stream())
    if code == 10002:
        add_launches(-1)
        return None
    _check(code, "branch_sum_rmsnorm")
    return out


# ------------------------------------------------------------------------------------------------
# Operations of layers whose projections pass a short convolution over time, and of norms on a part of a stacked
# projection (csrc/short_conv.cu, stream_ops.cu).
def short_conv(u: torch.Tensor, weight: torch.Tensor, states: torch.Tensor | None, state_slots: torch.Tensor, ctx, channels: int | None = None) -> torch.Tensor:
    """A causal convolution over time on each of the first ``channels`` columns of ``u [N, >= channels]`` (rows may have a
    pitch): ``y_t = sum_j weight[:, j] * u_(t - taps + 1 + j)`` within every request, ``weight [channels, taps]`` float32.
    What lies before a request's first row of this step is read from ``states[state_slots[r]]`` (``[slots, taps - 1,
    channels]`` float32: the last rows that earlier steps brought, zeros at a request's start), which is then moved on
    to the last ``taps - 1`` rows after this step.  A step in which no request brings more than 16 tokens
    (``ctx.max_query_len``) is one launch that walks every request's rows; the sums have the same order either way.
    Returns ``y [N, channels]`` float32."""
    c = int(channels) if channels is not None else weight.shape[0]
    taps = weight.shape[1]
    _need(u.dim() == 2 and u.stride(1) == 1 and u.shape[1] >= c, "short_conv: u [N, >= channels]")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == c and 1 <= taps <= 16, "short_conv: weight is float32 [channels, taps], taps up to 16")
    if taps > 1:
        _need(states is not None and states.dtype == torch.float32 and states.is_contiguous() and tuple(states.shape[1:]) == (taps - 1, c), "short_conv: states [slots, taps - 1, channels] float32")
    _i32(state_slots, "state_slots")
    out = torch.empty((u.shape[0], c), dtype=torch.float32, device=u.device)
    code = _launch("llm_short_conv", _ptr(u), _code(u.dtype), u.stride(0), _ptr(weight), _ptr(states), _ptr(state_slots), _ptr(ctx.token_request),
                   _ptr(ctx.cu_tokens), _ptr(out), out.stride(0), u.shape[0], ctx.num_requests, c, taps, int(getattr(ctx, "max_query_len", 0) or 0), _stream())
    _check(code, "short_conv")
    add_launches(int(taps > 1 and not 0 < int(getattr(ctx, "max_query_len", 0) or 0) <= 16))
    return out


def row_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` row by row for ``x [N, C]`` whose rows may have a pitch (a run of columns of a
    stacked projection); statistics in 32-bit; a contiguous ``[N, C]`` in ``out_dtype`` (default: the type of ``x``)."""
    _need(x.dim() == 2 and x.stride(1) == 1 and weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == x.shape[1],
          "row_rmsnorm: x [N, C] with unit inner stride, weight float32 [C]")
    out_dtype = out_dtype or x.dtype
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    code = _launch("llm_row_rmsnorm", _ptr(x), _code(x.dtype), x.stride(0), _ptr(weight), float(eps), _ptr(out), _code(out_dtype), out.stride(0),
                   x.shape[0], x.shape[1], _stream())
    _check(code, "row_rmsnorm")
    return out
