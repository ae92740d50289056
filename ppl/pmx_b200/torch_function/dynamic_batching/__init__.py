"""`pmx_llm.torch_function.dynamic_batching` operators covered by this package.

`multi_head_cache_attention` keeps the signature, output layout and ONNX custom-op export of
the reference operator (torch_function/dynamic_batching/MultiHeadCacheAttention.py:13-147) for
DECODE steps: every sequence of the batch contributes one new token, cache_mode 0 (any of
the four cache layouts), no cache quantisation, no explicit mask, no ALiBi.  Where the
reference loops over the sequences in Python -- storing the new key / value, gathering the
cached rows (KeyValueCache.py:86-138) and running one small attention per sequence
(MultiHeadAttention.py:76-108) -- this is one split-KV launch plus a merge over the whole
batch.  Calls outside that slice (prefill steps, paged or quantised caches, masks) raise
NotImplementedError: the caller keeps the reference operator for those.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..._cabi import lib, check, ptr, stream_of, workspace, DTYPE_CODE
from ..moe import _require_cuda


def set_decode_attention_kernel(kind: str) -> str:
    """Which kernel the decode-step attention runs: "mma" (default; tensor-core products on
    tiles staged in shared memory) or "simt" (CUDA cores, loads straight into registers).
    Process-wide; returns the previous choice."""
    names = ("mma", "simt")
    return names[lib.pmx_decode_cache_attention_set_kernel(names.index(kind))]


def cache_strides(cache: torch.Tensor, cache_layout: int, num_layer: int, layer_idx: int):
    """-> (layer_offset, row_stride, kv_stride, head_stride, total_rows) in elements for the
    four cache layouts of cache_mode 0 (Pipeline.py:80-89 of the Mixtral model):
      0: [rows, layers, 2, heads, d]   1: [layers, rows, 2, heads, d]
      2: [layers, 2, rows, heads, d]   3: [layers, 2, heads, rows, d]"""
    if cache.dim() != 5 or not cache.is_contiguous():
        raise ValueError("the cache must be a contiguous 5-d tensor")
    d = cache.shape[-1]
    if cache_layout == 0:
        rows, layers, two, heads, _ = cache.shape
        st = (layer_idx * 2 * heads * d, layers * 2 * heads * d, heads * d, d)
    elif cache_layout == 1:
        layers, rows, two, heads, _ = cache.shape
        st = (layer_idx * rows * 2 * heads * d, 2 * heads * d, heads * d, d)
    elif cache_layout == 2:
        layers, two, rows, heads, _ = cache.shape
        st = (layer_idx * 2 * rows * heads * d, heads * d, rows * heads * d, d)
    elif cache_layout == 3:
        layers, two, heads, rows, _ = cache.shape
        st = (layer_idx * 2 * heads * rows * d, d, heads * rows * d, rows * d)
    else:
        raise ValueError(f"unsupported cache_layout: {cache_layout}")
    if two != 2 or layers != num_layer or not 0 <= layer_idx < layers:
        raise ValueError(f"cache shape {tuple(cache.shape)} does not fit layout {cache_layout} with {num_layer} layers")
    return st + (rows,)


class MultiHeadCacheAttention(torch.autograd.Function):
    """opmx.dynamic_batching::MultiHeadCacheAttention."""

    @staticmethod
    def symbolic(g, query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos, decoding_batches,
                 max_seqlen, max_kvlen, cache, scale, attn_mask, num_heads: int, head_dim: int,
                 is_causal: bool = True, is_alibi: bool = False, num_kv_heads: int = 0, num_layer: int = 1,
                 layer_idx: int = 0, quant_bit: int = 0, quant_group: int = 8, cache_mode: int = 0,
                 cache_layout: int = 0, page_size: int = 128):
        args = [query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos, decoding_batches,
                max_seqlen, max_kvlen, cache]
        if attn_mask is not None:
            args += [scale, attn_mask]
        elif scale is not None:
            args += [scale]
        out = g.op("opmx.dynamic_batching::MultiHeadCacheAttention", *args, num_heads_i=num_heads,
                   head_dim_i=head_dim, is_causal_i=is_causal, is_alibi_i=is_alibi, num_kv_heads_i=num_kv_heads,
                   num_layer_i=num_layer, layer_idx_i=layer_idx, quant_bit_i=quant_bit, quant_group_i=quant_group,
                   cache_mode_i=cache_mode, cache_layout_i=cache_layout, page_size_i=page_size)
        return out.setTypeAs(query)

    @staticmethod
    def forward(ctx, query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos,
                decoding_batches, max_seqlen, max_kvlen, cache, scale, attn_mask, num_heads: int, head_dim: int,
                is_causal: bool = True, is_alibi: bool = False, num_kv_heads: int = 0, num_layer: int = 1,
                layer_idx: int = 0, quant_bit: int = 0, quant_group: int = 8, cache_mode: int = 0,
                cache_layout: int = 0, page_size: int = 128):
        if torch.onnx.is_in_onnx_export():
            return query
        _require_cuda("multi_head_cache_attention", query=query, current_key=current_key, current_value=current_value,
                      cache=cache, cachestarts=cachestarts, start_pos=start_pos)
        B = query.shape[0]
        why = None
        if int(max_seqlen.reshape(-1)[0]) != 1 or seqstarts.numel() != B + 1 or int(decoding_batches.reshape(-1)[0]) != B:
            why = "a step that is not a pure decode step (one new token per sequence)"
        elif cache_mode != 0:
            why = f"cache_mode {cache_mode}"
        elif quant_bit != 0:
            why = "a quantised cache"
        elif is_alibi or (attn_mask is not None and attn_mask.numel() > 0):
            why = "an explicit mask or ALiBi"
        if why is not None:
            raise NotImplementedError(f"multi_head_cache_attention: {why} is outside what this implementation "
                                      "covers; use the reference operator for it")
        kv_heads = num_kv_heads or num_heads
        if tuple(query.shape) != (B, num_heads, head_dim) or tuple(current_key.shape) != (B, kv_heads, head_dim) \
                or current_value.shape != current_key.shape:
            raise ValueError("multi_head_cache_attention: query must be [B, num_heads, head_dim] and the new key / "
                             "value [B, num_kv_heads, head_dim]")
        if query.dtype != cache.dtype or current_key.dtype != cache.dtype:
            raise TypeError("multi_head_cache_attention: query, key, value and cache must share one dtype")
        try:
            code = DTYPE_CODE[query.dtype]
        except KeyError:
            raise TypeError(f"multi_head_cache_attention: dtype {query.dtype} is not supported") from None
        layer_off, row_stride, kv_stride, head_stride, _ = cache_strides(cache, cache_layout, num_layer, layer_idx)
        dev = query.device
        q, kc, vc = query.contiguous(), current_key.contiguous(), current_value.contiguous()
        cs = cachestarts.to(device=dev, dtype=torch.int64).contiguous()
        sp = start_pos.to(device=dev, dtype=torch.int64).contiguous()
        kvmax = int(max_kvlen.reshape(-1)[0])
        out = torch.empty_like(q)
        nbytes = lib.pmx_decode_cache_attention_workspace_bytes(B, num_heads, kv_heads, head_dim, kvmax)
        ws = workspace(nbytes, dev)
        with torch.cuda.device(dev):
            check(lib.pmx_decode_cache_attention(ptr(q), ptr(kc), ptr(vc), ptr(cache), ptr(cs), ptr(sp), ptr(out), B,
                                                 num_heads, kv_heads, head_dim, layer_off, row_stride, kv_stride,
                                                 head_stride, kvmax, code, ptr(ws), ws.numel(), stream_of(q)))
        return out


def multi_head_cache_attention(query: torch.Tensor, current_key: torch.Tensor, current_value: torch.Tensor,
                               seqstarts: torch.Tensor, kvstarts: torch.Tensor, cachestarts: torch.Tensor,
                               start_pos: torch.Tensor, decoding_batches: torch.Tensor, max_seqlen: torch.Tensor,
                               max_kvlen: torch.Tensor, cache: torch.Tensor, scale: Optional[torch.Tensor],
                               attn_mask: Optional[torch.Tensor], num_heads: int, head_dim: int,
                               is_causal: bool = True, is_alibi: bool = False, num_kv_heads: int = 0,
                               num_layer: int = 1, layer_idx: int = 0, quant_bit: int = 0, quant_group: int = 8,
                               cache_mode: int = 0, cache_layout: int = 0, page_size: int = 128) -> torch.Tensor:
    """Signature of torch_function/dynamic_batching/MultiHeadCacheAttention.py:133-147.
    -> [B, num_heads, head_dim]; the new keys and values are written into `cache` in place."""
    return MultiHeadCacheAttention.apply(query, current_key, current_value, seqstarts, kvstarts, cachestarts,
                                         start_pos, decoding_batches, max_seqlen, max_kvlen, cache, scale, attn_mask,
                                         num_heads, head_dim, is_causal, is_alibi, num_kv_heads, num_layer, layer_idx,
                                         quant_bit, quant_group, cache_mode, cache_layout, page_size)
