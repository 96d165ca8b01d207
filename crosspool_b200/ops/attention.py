"""Attention-side operators on the in-tree kernels: q/k-norm + RoPE + paged KV write, paged decode
attention (split-KV) and chunked causal prefill attention over the paged cache, embedding gather and
greedy sampling. The reference owns none of these (SGLang/FlashInfer do, pyproject.toml:17-35); the
oracles are plain fp32 PyTorch restatements in ``tests/``.
"""

from __future__ import annotations

import ctypes as C
import os
import math

import torch

from .. import native


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  positions: torch.Tensor, slots: torch.Tensor, *, q_heads: int, kv_heads: int, head_dim: int,
                  theta: float, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                  eps: float = 1e-6) -> None:
    """qkv ``[rows, (q+2kv)*d]`` → RoPE'd q in ``q_out`` and k/v scattered to the paged cache."""
    a = native.RopeArgs()
    a.qkv, a.q_out = qkv.data_ptr(), q_out.data_ptr()
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.q_norm_weight = q_norm.data_ptr() if q_norm is not None else None
    a.k_norm_weight = k_norm.data_ptr() if k_norm is not None else None
    assert positions.dtype == torch.int32 and slots.dtype == torch.int32
    a.positions, a.slots = positions.data_ptr(), slots.data_ptr()
    a.rows, a.ld_qkv = qkv.shape[0], qkv.stride(0)
    a.q_heads, a.kv_heads, a.head_dim = q_heads, kv_heads, head_dim
    a.eps, a.log2_theta = eps, math.log2(theta)
    native.check(native.kernels().xp_rope_kv(C.byref(a), _stream(qkv.device)), "xp_rope_kv")


def decode_splits(batch: int, kv_heads: int, max_len: int) -> int:
    return native.kernels().xp_decode_attn_splits(batch, kv_heads, max_len)


# Which prefill kernel runs when the caller does not say: "umma" (tcgen05 tensor cores, TMEM accumulators; shapes it
# does not cover fall back to "mma"), "mma" (TMA-fed mma.sync kernel) or "simple" (plain mma.sync kernel).
# "umma-alt" is the tcgen05 kernel with the other route for the probabilities (tensor memory <-> shared memory).
# XPOOL_PREFILL_KERNEL selects one, e.g. to bisect a numerical difference.
PREFILL_KERNELS = {"umma": 0, "simple": 1, "mma": 2, "umma-alt": 0x100}
PREFILL_KERNEL_DEFAULT = os.environ.get("XPOOL_PREFILL_KERNEL", "umma")


def decode_plan(batch: int, kv_heads: int, max_len: int) -> tuple[int, int]:
    """(num_splits, chunk_tokens) for a decode batch.

    A CTA covers one (sequence, KV head, slice); its fixed cost (first TMA round trip, cross-warp merge,
    partial write + merge kernel) is amortised best by long slices, so sequences are only cut when there
    are too few (sequence, head) pairs to fill the 148 SMs a few times over. Measured on B200 (16 q / 8 kv
    heads, d 128, lengths 128-2048): batch 256 reaches 0.92 of copy bandwidth unsplit, 0.87 with 512-token
    slices, 0.77 with 256-token slices."""
    pairs = batch * kv_heads
    if pairs >= 1024 or max_len <= 512:
        return 1, 0
    chunk = 1024 if pairs >= 256 else 512 if pairs >= 64 else 256
    if max_len <= chunk:
        return 1, 0
    return (max_len + chunk - 1) // chunk, chunk


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, *, out: torch.Tensor | None = None, num_splits: int = 0,
                 ws: torch.Tensor | None = None, scale: float | None = None, max_len: int | None = None,
                 chunk_tokens: int = 0, force_simt: bool = False) -> torch.Tensor:
    """q ``[batch, q_heads, d]`` against caches ``[pages, page, kv_heads, d]``.

    Runs the tensor-core kernel (TMA-fed ``mma`` tiles) whenever pages hold a multiple of 16 tokens
    and at most 16 query heads share a KV head; ``force_simt`` selects the plain kernel."""
    batch, q_heads, d = q.shape
    page_size, kv_heads = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty_like(q)
    if num_splits <= 0:
        num_splits = decode_splits(batch, kv_heads, max_len or block_table.shape[1] * page_size)
    if num_splits > 1 and ws is None:
        ws = torch.empty(batch * q_heads * num_splits * (d + 2), dtype=torch.float32, device=q.device)
    a = native.DecodeAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    a.ws = ws.data_ptr() if ws is not None else None
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    a.block_table, a.seq_lens = block_table.data_ptr(), seq_lens.data_ptr()
    a.batch, a.q_heads, a.kv_heads, a.head_dim = batch, q_heads, kv_heads, d
    a.page_size, a.max_blocks, a.num_splits = page_size, block_table.stride(0), num_splits
    a.scale = scale if scale is not None else d ** -0.5
    a.chunk_tokens = chunk_tokens
    a.num_pages = k_cache.shape[0] if k_cache.is_contiguous() and v_cache.is_contiguous() else 0
    a.force_simt = int(force_simt)
    from .gemm import status_words

    a.status = status_words(q.device).data_ptr()
    native.check(native.kernels().xp_decode_attn(C.byref(a), _stream(q.device)), "xp_decode_attn",
                 2 if num_splits > 1 else 1)
    return out


def paged_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                  q_starts: torch.Tensor, q_lens: torch.Tensor, ctx_lens: torch.Tensor, max_q_len: int, *,
                  out: torch.Tensor | None = None, scale: float | None = None,
                  force_simple: bool | str | None = None) -> torch.Tensor:
    """Causal attention of packed chunk queries ``[total_q, q_heads, d]`` over the paged cache.

    Runs the tcgen05 kernel (S and O in tensor memory, TMA-fed Q/K/V, the heads of a KV group packed into 128-row
    tiles) when pages hold a power-of-two number of at least 16 tokens and 1, 2, 4, 8 or 16 query heads share a KV
    head. ``force_simple``: True or ``"simple"`` selects the plain kernel, ``"mma"`` the TMA-fed mma.sync kernel."""
    _, q_heads, d = q.shape
    page_size, kv_heads = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty_like(q)
    a = native.PrefillAttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    a.block_table = block_table.data_ptr()
    a.q_starts, a.q_lens, a.ctx_lens = q_starts.data_ptr(), q_lens.data_ptr(), ctx_lens.data_ptr()
    a.num_seqs, a.max_q_len = q_lens.shape[0], max_q_len
    a.q_heads, a.kv_heads, a.head_dim = q_heads, kv_heads, d
    a.page_size, a.max_blocks = page_size, block_table.stride(0)
    a.scale = scale if scale is not None else d ** -0.5
    a.num_pages = k_cache.shape[0] if k_cache.is_contiguous() and v_cache.is_contiguous() else 0
    which = PREFILL_KERNEL_DEFAULT if force_simple in (None, False) else ("simple" if force_simple is True else force_simple)
    a.force_simple = PREFILL_KERNELS[which]
    a.total_q = q.shape[0]
    from .gemm import status_words

    a.status = status_words(q.device).data_ptr()
    native.check(native.kernels().xp_prefill_attn(C.byref(a), _stream(q.device)), "xp_prefill_attn")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows, hidden = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty(rows, hidden, dtype=table.dtype, device=table.device)
    native.check(native.kernels().xp_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), rows, hidden,
                                               table.shape[0], _stream(table.device)), "xp_embedding")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    native.check(native.kernels().xp_argmax(logits.data_ptr(), int(logits.dtype == torch.float32), out.data_ptr(),
                                            rows, vocab, logits.stride(0), _stream(logits.device)), "xp_argmax")
    return out


def sample(logits: torch.Tensor, temps: torch.Tensor, seeds: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row from ``softmax(logits / temperature)`` (Gumbel-max); rows with temperature 0 are
    greedy. ``temps`` fp32 ``[rows]``; ``seeds`` int32 ``[rows, 2]`` = (request seed, step): the same pair
    always gives the same token."""
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    assert temps.dtype == torch.float32 and seeds.dtype == torch.int32 and seeds.shape[-1] == 2
    native.check(native.kernels().xp_sample(logits.data_ptr(), int(logits.dtype == torch.float32), temps.data_ptr(),
                                            seeds.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0),
                                            _stream(logits.device)), "xp_sample")
    return out
