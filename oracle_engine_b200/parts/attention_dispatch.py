"""Which attention kernels a step uses: chosen by precision, head size and whether the
step is a prompt or single decoded tokens; never by the data.

float32, and head sizes the tensor-core kernels do not take, use the one-path kernel of
csrc/attention.cu; bfloat16 uses the tensor-core prefill kernel and the split-KV decode
kernel of csrc/attention_mma.cu.
"""
from __future__ import annotations

import torch

from ..csrc import ops


def mixer_core(rt, out, qkv, cos, sin, cache, ctx, H, KVH, hd, window, scale, owns_cache) -> None:
    """Rotation, cache write and attention of one attention mixer for the step's tokens."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores and ctx.all_decode and ctx.n_tokens == ctx.n_seqs:
        from ..csrc import ops_tc
        # One CTA (or, for few long sequences, one cluster of CTAs) per (sequence, KV head) whose warps
        # split the keys: one launch for rotation, cache write, attention and the merge, no scratch in
        # global memory.  Every model whose groups have up to 16 heads of a multiple of 32 dims goes here.
        if ops_tc.decode_uses_warps(ctx.n_seqs, getattr(ctx, "context_class", 0), hd, H, KVH):
            ops_tc.attention_decode_warps(out, qkv, cos, sin, cache.kv, cache.tables, ctx, H, KVH, hd, window,
                                          scale, owns_cache)
            return
        # Larger groups: one kernel when the batch alone fills the GPU (no split over the keys), else
        # rotation, the kernel that splits the keys over CTAs, and a merge.
        if ops_tc.decode_fused_supported(hd, H, KVH) and \
                ops_tc.decode_splits_for(ctx.n_seqs, KVH, cache.tables, getattr(ctx, "context_class", 0), hd) == 1:
            ops_tc.attention_decode_fused(out, qkv, cos, sin, cache.kv, cache.tables, ctx, H, KVH, hd, window,
                                          scale, owns_cache, n_splits=1)
            return
    rope_and_cache(rt, qkv, cos, sin, cache, ctx, H, KVH, hd, owns_cache)
    attend(rt, out, qkv, cache, ctx, H, KVH, hd, window, scale)


def rope_and_cache(rt, qkv, cos, sin, cache, ctx, H, KVH, hd, owns_cache) -> None:
    ops.rope_kv_write(qkv, cos, sin, cache.kv if owns_cache else None, cache.tables, ctx.tok_seq,
                      ctx.tok_pos, H, KVH, hd, owns_cache)


def attend(rt, out, qkv, cache, ctx, H, KVH, hd, window, scale, sink: bool = False) -> None:
    """sink: the softmax's denominator gets one added (a key of score 0 without a value), in every kernel."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.attention_supported(hd, H, KVH):
            ops_tc.attention(out, qkv, cache.kv, cache.tables, ctx, H, KVH, hd, window, scale, sink)
            return
    ops.attn_paged(out, qkv, cache.kv, cache.tables, ctx.tok_seq, ctx.tok_pos, H, KVH, hd, window, scale, sink)


def split_mixer_core(rt, out, qkv, cos, sin, rot, kcache, vcache, tables, ctx, H, G, dk, dv, window, scale, cap) -> None:
    """Rotation, cache write and attention of an attention mixer whose keys and values have head sizes of their
    own and lie in two cache tensors, with a cap on the scores (parts/capped_attention.py)."""
    ops.rope_split_kv_write(qkv, cos, sin, rot, kcache, vcache, tables, ctx.tok_seq, ctx.tok_pos, H, G, dk, dv, True)
    split_attend(rt, out, qkv, kcache, vcache, tables, ctx, H, G, dk, dv, window, scale, cap)


def split_attend(rt, out, q, kcache, vcache, tables, ctx, H, G, dk, dv, window, scale, cap, sinks=None,
                 unrotate=None) -> None:
    """Attention of queries that are turned already over keys and values that lie in two cache tensors; `sinks`
    (float32 [H] or None): a learned score per head that joins the softmax's denominator without key or value;
    `unrotate` ((cos, sin) tables [positions, dv/2] or None): every head's result is turned back by its query's
    position inside the kernel that stores it."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.attention_split_supported(dk, dv, H, G):
            ops_tc.attention_split(out, q, kcache, vcache, tables, ctx, H, G, dk, dv, window, scale, cap, sinks, unrotate)
            return
    ops.attn_split(out, q, kcache, vcache, tables, ctx.tok_seq, ctx.tok_pos, H, G, dk, dv, window, scale, cap, sinks,
                   unrotate)


def latent_core(rt, out, qfull, rows, tables, ctx, H, r, rd, scale) -> None:
    """Attention of absorbed queries [T, H (r + rd)] over a cache of latent rows [r + rd]; out [T, H r] gets each
    head's weighted sum of the latents (parts/latent_attention.py)."""
    if rt.dtype == torch.bfloat16 and rt.tensor_cores:
        from ..csrc import ops_tc
        if ops_tc.attention_latent_supported(H, r, rd):
            ops_tc.attention_latent(out, qfull, rows, tables, ctx, H, r, rd, scale)
            return
    ops.attn_latent(out, qfull, rows, tables, ctx, H, r, rd, scale)
