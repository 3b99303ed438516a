"""Two-stage mixture-of-experts GEMM: the operator surface of the reference's
``kernels/moe/moe_gemm_2stage`` (gemm1.py:541-580 ``compile_moe_gemm1``,
gemm2.py:595-643 ``compile_moe_gemm2``, moe_reduce.py:164-205
``compile_moe_reduction``) bound to the grouped kernels of libflyb200.

    exe = compile_moe_gemm1(model_dim=.., inter_dim=.., experts=.., topk=.., tile_m=.., tile_n=.., tile_k=..,
                            doweight_stage1=False, out_dtype="bf16", in_dtype="fp8")
    exe(out, x, w1_shuffled, scale_x, scale_w1, sorted_token_ids, sorted_expert_ids, sorted_weights,
        num_valid_ids, tokens, inter_dim, model_dim, blocks, stream)          # -> None, writes out

The positional arguments are the reference's
(tests/kernels/test_moe_gemm_2stage.py:161-193).  ``w`` is
``shuffle_weight(w_q)`` of the ``[experts, rows, K]`` weights: one B200 image
per expert.  ``tile_m`` is the routing block size the sorted ids were padded
to; ``tile_n`` / ``tile_k`` are validated as the reference does and are
otherwise hints (a CTA always takes two 128-channel weight tiles and 128-byte
k-blocks).  ``in_dtype`` "fp8", "int8", "int8smooth" and "int4" are built.  "int4"
is W4A8 (tests/kernels/test_moe_gemm_2stage.py:64-79,212-220): int8 activations and
weights quantised to [-8, 7], passed as the preshuffled int8 image packed two
values per byte (``pack_shuffled_int8_to_packed_int4``).  The tensor core has no
4-bit integer kind, so the launcher expands a packed weight tensor back to its
int8 image the first time it sees it (cached by address; ``forget_weights``
drops an entry) and runs the int8 kernels: same results as the reference, the
weight stream of int8.

``moe_sorting`` builds the routing table the kernels consume (layout:
tests/kernels/test_moe_gemm_2stage.py:99-137): on CUDA tensors with the
library's counting-sort kernels, on CPU tensors with torch ops.
"""

from __future__ import annotations

from typing import Tuple

import torch

from .... import _lib
from ...gemm.preshuffle_gemm import _stream_handle

_OUT = {
    "f16": (_lib.OUT_FP16, torch.float16),
    "fp16": (_lib.OUT_FP16, torch.float16),
    "half": (_lib.OUT_FP16, torch.float16),
    "bf16": (_lib.OUT_BF16, torch.bfloat16),
    "bfloat16": (_lib.OUT_BF16, torch.bfloat16),
    "f32": (_lib.OUT_F32, torch.float32),
    "fp32": (_lib.OUT_F32, torch.float32),
    "float": (_lib.OUT_F32, torch.float32),
}
_IN = {
    "fp8": (_lib.DT_FP8, torch.float8_e4m3fn),
    "int8": (_lib.DT_INT8, torch.int8),
    # int8 with per-route ("smooth-quantised") activations: stage 1 reads x and scale_x
    # slot-major, [topk * tokens, ...] with row = slot * tokens + token; stage 2 is plain int8
    "int8smooth": (_lib.DT_INT8, torch.int8),
    # W4A8: int8 activations, weights in [-8, 7] passed packed two per byte and expanded once to the int8 image
    "int4": (_lib.DT_INT8, torch.int8),
}


def pack_shuffled_int8_to_packed_int4(x_shuf_i8: torch.Tensor) -> torch.Tensor:
    """Pack a preshuffled int8 weight image with values in [-8, 7] two per byte, as the reference's
    helper does (tests/kernels/test_moe_gemm_2stage.py:64-79): every 8 consecutive values v0..v7
    become 4 bytes, byte j = (v_j & 15) | (v_{j+4} << 4)."""
    u = (x_shuf_i8.contiguous().view(-1).to(torch.int16) & 0xF).to(torch.uint8).view(-1, 8)
    return (u[:, :4] | (u[:, 4:] << 4)).contiguous().view(-1).view(torch.int8)


def unpack_packed_int4_to_shuffled_int8(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_shuffled_int8_to_packed_int4`: 4 bytes -> 8 sign-extended int8 values."""
    b = packed.contiguous().view(-1).view(torch.uint8).view(-1, 4)
    nib = torch.cat([b & 0xF, b >> 4], dim=1).to(torch.int16)  # v0..v3 from the low nibbles, v4..v7 from the high ones
    return ((nib ^ 8) - 8).to(torch.int8).view(-1)
_REFERENCE_IN_DTYPES = ("fp8", "int8", "int8smooth", "int4")


def moe_sorting(
    topk_ids: torch.Tensor, topk_weights: torch.Tensor, *, num_experts: int, block_size: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Routing table for the two GEMM stages: ``(sorted_ids, sorted_weights,
    sorted_expert_ids, num_tokens_post_pad)``.

    The (token, slot) pairs are grouped by expert in ascending (token, slot)
    order, every group padded to a multiple of ``block_size``; a sorted id is
    ``(slot << 24) | token``, padding is ``(topk << 24) | tokens``;
    ``sorted_expert_ids[b]`` is the expert of block ``b`` (-1 past the end);
    ``num_tokens_post_pad = [rows in use, tokens]``.
    """
    tokens, topk = topk_ids.shape
    dev = topk_ids.device
    e, bs = int(num_experts), int(block_size)
    max_padded = int(topk_ids.numel() + e * bs - topk)
    max_blocks = (max_padded + bs - 1) // bs
    if topk_ids.is_cuda:
        # device kernels (flyb200_moe_sorting): no host synchronisation, capturable
        ids32 = topk_ids.to(torch.int32).contiguous()
        w32 = topk_weights.to(torch.float32).contiguous()
        sorted_ids = torch.empty((max_padded,), dtype=torch.int32, device=dev)
        sorted_weights = torch.empty((max_padded,), dtype=torch.float32, device=dev)
        sorted_expert_ids = torch.empty((max_blocks,), dtype=torch.int32, device=dev)
        post_pad = torch.empty((2,), dtype=torch.int32, device=dev)
        counts = torch.empty((e,), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(
                _lib.load().flyb200_moe_sorting(
                    ids32.data_ptr(), w32.data_ptr(), tokens, topk, e, bs, sorted_ids.data_ptr(), sorted_weights.data_ptr(),
                    sorted_expert_ids.data_ptr(), post_pad.data_ptr(), counts.data_ptr(),
                    torch.cuda.current_stream(dev).cuda_stream,
                ),
                "moe_sorting",
            )
        return sorted_ids, sorted_weights, sorted_expert_ids, post_pad
    flat = topk_ids.reshape(-1).to(torch.int64)
    flat = torch.where((flat >= 0) & (flat < e), flat, torch.full_like(flat, e))  # ids outside [0, e) are dropped
    order = torch.sort(flat, stable=True).indices  # by expert, then (token, slot)
    counts = torch.bincount(flat, minlength=e + 1)[:e]
    padded = (counts + bs - 1) // bs * bs
    starts = torch.cumsum(padded, 0) - padded
    first = torch.cumsum(counts, 0) - counts
    order = order[: int(counts.sum())]
    expert_of = flat[order]
    dest = starts[expert_of] + (torch.arange(order.numel(), device=dev) - first[expert_of])
    sorted_ids = torch.full((max_padded,), (topk << 24) | tokens, dtype=torch.int32, device=dev)
    sorted_weights = torch.zeros((max_padded,), dtype=torch.float32, device=dev)
    tok = (order // topk).to(torch.int32)
    slot = (order % topk).to(torch.int32)
    sorted_ids[dest] = (slot << 24) | tok
    sorted_weights[dest] = topk_weights.reshape(-1).to(torch.float32)[order]
    blocks_per = padded // bs
    sorted_expert_ids = torch.full((max_blocks,), -1, dtype=torch.int32, device=dev)
    total_blocks = int(blocks_per.sum())
    sorted_expert_ids[:total_blocks] = torch.repeat_interleave(
        torch.arange(e, device=dev, dtype=torch.int32), blocks_per
    )
    num_tokens_post_pad = torch.tensor([int(padded.sum()), tokens], dtype=torch.int32, device=dev)
    return sorted_ids, sorted_weights, sorted_expert_ids, num_tokens_post_pad


class _MoeStage:
    """Shared launcher: gathers the activation rows into sorted order, then runs the grouped GEMM."""

    def __init__(self, stage, model_dim, inter_dim, experts, topk, tile_m, in_dtype, out_dtype, doweight, accumulate):
        self.stage = stage
        self.model_dim, self.inter_dim = int(model_dim), int(inter_dim)
        self.experts, self.topk, self.tile_m = int(experts), int(topk), int(tile_m)
        self.in_dtype, self.out_dtype = in_dtype, out_dtype
        self.doweight, self.accumulate = bool(doweight), bool(accumulate)
        self._dt, self._torch_in = _IN[in_dtype]
        self._out, self._torch_out = _OUT[out_dtype]
        self._k = self.model_dim if stage == 1 else self.inter_dim
        self._slot_major = stage == 1 and in_dtype == "int8smooth"
        self._gather_mode = (2 if self._slot_major else 0) if stage == 1 else 1  # how a sorted row finds its activation row
        self._scratch: dict = {}
        self._retired: list = []
        self._w4_expanded: dict = {}  # (data_ptr, numel) of a packed int4 weight tensor -> its int8 image

    def _weights_for_kernel(self, w: torch.Tensor, w_elems: int) -> torch.Tensor:
        """W4A8: a tensor of w_elems / 2 bytes is the packed form; expand it once.  Anything else passes through."""
        if self.in_dtype != "int4" or w.numel() != w_elems // 2:
            return w
        key = (w.data_ptr(), w.numel())
        img = self._w4_expanded.get(key)
        if img is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("moe_gemm: packed int4 weights are expanded on first use; call the launcher once "
                                   "before capturing a CUDA graph")
            img = unpack_packed_int4_to_shuffled_int8(w)
            self._w4_expanded[key] = img
        return img

    def forget_weights(self, w: torch.Tensor) -> None:
        """Drop the cached int8 image of a packed int4 weight tensor (its contents changed in place)."""
        self._w4_expanded.pop((w.data_ptr(), w.numel()), None)

    def _sorted_buffers(self, device, rows, stream=0):
        """Gathered activation rows and their scales, one pair per (device, stream): two launches
        on different streams must not share them.  A buffer that has to grow is replaced but
        never freed (a kernel still running or a captured graph may hold its address), and
        growing inside a stream capture is refused: run the shape once before capturing."""
        key = (device.index, stream or 0)
        buf = self._scratch.get(key)
        if buf is None or buf[0].shape[0] < rows:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("moe_gemm: the gather scratch for this shape does not exist yet; call the launcher "
                                   "once on this stream before capturing a CUDA graph")
            if buf is not None:
                self._retired.append(buf)
            buf = (
                torch.empty((rows, self._k), dtype=torch.uint8, device=device),
                torch.empty((rows,), dtype=torch.float32, device=device),
            )
            self._scratch[key] = buf
        return buf

    def __call__(
        self, out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights, num_valid_ids,
        tokens, dim0, dim1, blocks, stream=None,
    ):
        self._check(out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights, num_valid_ids,
                    tokens, dim0, dim1, blocks)
        return self._launch(out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights,
                            num_valid_ids, int(tokens), int(blocks), stream)

    def _compile_for(self, *args):
        """``flyc.compile(exe, *args)``: check the example arguments once and return a callable with the
        same signature that goes straight to the library, as the reference's compiled function checks
        nothing per call (python/flydsl/compiler/jit_executor.py:185-214)."""
        if len(args) >= 13:
            self._check(*args[:13])
        stage = self

        def compiled(out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights, num_valid_ids,
                     tokens, dim0, dim1, blocks, stream=None):
            return stage._launch(out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights,
                                 num_valid_ids, int(tokens), int(blocks), stream)

        return compiled

    def _check(self, out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights, num_valid_ids,
               tokens, dim0, dim1, blocks):
        n_out, k = (self.inter_dim, self.model_dim) if self.stage == 1 else (self.model_dim, self.inter_dim)
        if (int(dim0), int(dim1)) != (n_out, k):
            raise ValueError(f"launch dims ({dim0}, {dim1}) do not match the compiled ({n_out}, {k})")
        tokens, blocks = int(tokens), int(blocks)
        for name, t in (("out", out), ("x", x), ("w", w), ("scale_x", scale_x), ("scale_w", scale_w)):
            if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous CUDA tensor")
        if out.dtype != self._torch_out:
            raise ValueError(f"out must be {self._torch_out}, got {out.dtype}")
        x_rows = tokens if (self.stage == 1 and not self._slot_major) else tokens * self.topk
        out_rows = tokens if (self.stage == 2 and self.accumulate) else tokens * self.topk
        w_rows = self.experts * (2 * self.inter_dim if self.stage == 1 else self.model_dim)
        if self.in_dtype == "int4" and w.numel() == w_rows * k // 2:
            w_need = w_rows * k // 2  # packed two values per byte
        else:
            w_need = w_rows * k
        need = (
            ("out", out, out_rows * n_out), ("x", x, x_rows * k), ("w", w, w_need),
            ("scale_x", scale_x, x_rows), ("scale_w", scale_w, w_rows),
            # the sorted ids are read up to num_valid_ids[0] only, which may end inside the last block
            ("sorted_token_ids", sorted_token_ids, (blocks - 1) * self.tile_m + 1), ("sorted_expert_ids", sorted_expert_ids, blocks),
            ("num_valid_ids", num_valid_ids, 1),
        )
        for name, t, n in need:
            if t.numel() < n:
                raise ValueError(f"{name} holds {t.numel()} elements, the launch needs {n}")
        if x.element_size() != 1 or w.element_size() != 1:
            raise ValueError("x and w must be 8-bit tensors")
        if scale_x.dtype != torch.float32 or scale_w.dtype != torch.float32:
            raise ValueError("scales must be float32")
        if sorted_token_ids.dtype != torch.int32 or sorted_expert_ids.dtype != torch.int32 or num_valid_ids.dtype != torch.int32:
            raise ValueError("routing tensors must be int32")
        if self.doweight and (sorted_weights is None or sorted_weights.numel() < sorted_token_ids.numel()):
            raise ValueError("sorted_weights is required when the routed weight is applied in this stage")

    def _launch(self, out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights, num_valid_ids,
                tokens, blocks, stream):
        if tokens == 0 or blocks == 0:
            return None
        dev = out.device
        if torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):
                return self._launch(out, x, w, scale_x, scale_w, sorted_token_ids, sorted_expert_ids, sorted_weights,
                                    num_valid_ids, tokens, blocks, stream)
        lib = _lib.load()
        s = _stream_handle(stream) or None
        rows = blocks * self.tile_m
        if self.in_dtype == "int4":
            w = self._weights_for_kernel(w, self.experts * (2 * self.inter_dim if self.stage == 1 else self.model_dim) * self._k)
        a_sorted, sa_sorted = self._sorted_buffers(dev, rows, s)
        a_ptr, sa_ptr, ids_ptr, nv_ptr = a_sorted.data_ptr(), sa_sorted.data_ptr(), sorted_token_ids.data_ptr(), num_valid_ids.data_ptr()
        rc = lib.flyb200_moe_gather_rows(a_ptr, sa_ptr, x.data_ptr(), scale_x.data_ptr(), ids_ptr, nv_ptr, tokens, self.topk,
                                         self._gather_mode, self._k, rows, s)
        if rc:
            _lib.check(rc, "moe_gather_rows")
        rc = lib.flyb200_moe_gemm(
            self.stage, out.data_ptr(), a_ptr, w.data_ptr(), sa_ptr, scale_w.data_ptr(), ids_ptr, sorted_expert_ids.data_ptr(),
            sorted_weights.data_ptr() if sorted_weights is not None and sorted_weights.numel() else None, nv_ptr,
            tokens, self.topk, self.experts, self.model_dim, self.inter_dim, self.tile_m, blocks, self._dt, self._out,
            int(self.doweight), int(self.accumulate), 1, s,
        )
        if rc:
            _lib.check(rc, "moe_gemm")
        return None


def _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, in_dtype, k):
    if in_dtype not in _REFERENCE_IN_DTYPES:
        raise ValueError(f"in_dtype must be 'fp8', 'int8', 'int8smooth', or 'int4', got {in_dtype!r}")
    if in_dtype not in _IN:
        raise ValueError(f"in_dtype={in_dtype!r} is not built for B200")
    if min(int(model_dim), int(inter_dim), int(experts), int(topk)) <= 0:
        raise ValueError("model_dim, inter_dim, experts and topk must be positive")
    if not (16 <= int(tile_m) <= 256 and int(tile_m) % 16 == 0):
        raise ValueError(f"tile_m must be a 16-multiple in [16,256], got {tile_m}")
    if not (64 <= int(tile_n) <= 256 and int(tile_n) % 64 == 0):
        raise ValueError(f"tile_n must be in [64,256] multiple of 64, got {tile_n}")
    if int(tile_k) not in (128, 256):
        raise ValueError(f"tile_k must be 128 or 256, got {tile_k}")
    if k % int(tile_k) != 0:
        raise ValueError(f"K={k} must be a multiple of tile_k={tile_k}")


def compile_moe_gemm1(
    *, model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, doweight_stage1, out_dtype="f16", in_dtype="fp8"
):
    """Stage 1 (gate-up + silu): ``out[token, slot, inter_dim] = silu(x.Wg) * (x.Wu)``."""
    if out_dtype not in ("f16", "bf16"):
        raise ValueError(f"out_dtype must be 'f16' or 'bf16', got {out_dtype!r}")
    _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, in_dtype, int(model_dim))
    if int(inter_dim) % 16 != 0:
        raise ValueError(f"inter_dim={inter_dim} must be a multiple of 16")
    return _MoeStage(1, model_dim, inter_dim, experts, topk, tile_m, in_dtype, out_dtype, doweight_stage1, False)


def compile_moe_gemm2(
    *, model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, doweight_stage2, out_dtype="f16",
    accumulate=True, in_dtype="fp8",
):
    """Stage 2 (down projection): atomic accumulation into ``[tokens, model_dim]``
    or per-(token, slot) rows ``[tokens * topk, model_dim]`` for a separate reduction."""
    out_s = str(out_dtype).strip().lower()
    if out_s not in _OUT:
        raise ValueError(f"out_dtype must be 'f16', 'bf16', or 'f32', got {out_dtype!r}")
    if (not bool(accumulate)) and _OUT[out_s][0] == _lib.OUT_F32:
        raise ValueError("compile_moe_gemm2(accumulate=False) only supports out_dtype in {'f16','bf16'}")
    _check_common(model_dim, inter_dim, experts, topk, tile_m, tile_n, tile_k, in_dtype, int(inter_dim))
    if int(model_dim) % 16 != 0:
        raise ValueError(f"model_dim={model_dim} must be a multiple of 16")
    return _MoeStage(2, model_dim, inter_dim, experts, topk, tile_m, in_dtype, out_s, doweight_stage2, accumulate)


def compile_moe_reduction(*, topk, model_dim, dtype_str="f16", use_mask=False, num_experts=0, out_dtype_str=None):
    """Top-k reduction ``Y[t, :] = sum_slot X[t, slot, :]``; returns
    ``launch(X, Y, expert_mask, topk_ids, m_tokens, stream)`` as the reference does.
    With ``use_mask`` slot k of token t counts only if ``expert_mask[topk_ids[t, k]] != 0``
    (int32 tensors; the expert-parallel validity mask): rows of masked routes are never read."""
    if dtype_str not in ("f16", "bf16") or (out_dtype_str or dtype_str) != dtype_str:
        raise ValueError("the reduction is built for f16 and bf16 with the output type of the input")
    code, tdt = _OUT[dtype_str]
    topk, model_dim, num_experts = int(topk), int(model_dim), int(num_experts)
    if model_dim % 2 != 0:
        raise ValueError("model_dim must be even")
    if use_mask and num_experts <= 0:
        raise ValueError("use_mask=True needs num_experts")

    def launch(X, Y, expert_mask, topk_ids, m_tokens, stream=None):
        m = int(m_tokens)
        if X.dtype != tdt or Y.dtype != tdt or not X.is_cuda or not Y.is_cuda:
            raise ValueError(f"X and Y must be CUDA tensors of {tdt}")
        if X.numel() < m * topk * model_dim or Y.numel() < m * model_dim:
            raise ValueError("X or Y is smaller than the launch needs")
        mask_ptr = ids_ptr = None
        if use_mask:
            for name, t, n in (("expert_mask", expert_mask, num_experts), ("topk_ids", topk_ids, m * topk)):
                if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.int32 or t.numel() < n or not t.is_contiguous():
                    raise ValueError(f"{name} must be a contiguous int32 CUDA tensor of at least {n} elements")
            mask_ptr, ids_ptr = expert_mask.data_ptr(), topk_ids.data_ptr()
        with torch.cuda.device(X.device):
            _lib.check(
                _lib.load().flyb200_moe_reduce(Y.data_ptr(), X.data_ptr(), m, topk, model_dim, code, mask_ptr, ids_ptr,
                                               num_experts, _stream_handle(stream) or None),
                "moe_reduce",
            )

    return launch


__all__ = ["compile_moe_gemm1", "compile_moe_gemm2", "compile_moe_reduction", "moe_sorting",
           "pack_shuffled_int8_to_packed_int4", "unpack_packed_int4_to_shuffled_int8"]
