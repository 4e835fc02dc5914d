"""The two operators of the decode attention path, with the reference's signatures.

``reshape_and_cache`` and ``paged_attention`` take the arguments of the ops that
MuxServe's ``PagedAttentionWithRoPE`` layer calls
(muxserve/flexserver/models/llama.py:138-147,160-161; the op source lives in the
un-vendored MuxServe-vLLM fork).  ``paged_attention_mixed`` is the extension
that serves several colocated models in one launch.  All three go through the
C ABI in ``libmuxb200.so`` on the current CUDA stream; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import AttnArgs, AttnMixedArgs, CacheWriteArgs, check, lib

HEAD_SIZE = 128
MAX_FUSED_NEW_TOKENS = 16  # new tokens per sequence that decode_attention appends in its own launch

_DTYPES = {torch.float16: _lib.MUX_DTYPE_F16, torch.bfloat16: _lib.MUX_DTYPE_BF16}
_workspaces = {}
launch_count = 0  # kernels enqueued by this module so far (cache write 1; attention 1, or 2 when partitioned)


def _dtype_code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DTYPES:
        raise TypeError(f"{name} must be float16 or bfloat16, got {t.dtype}")
    return _DTYPES[t.dtype]


def _require_cuda(**tensors) -> torch.device:
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (this op has no CPU implementation)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name} is on {t.device}, expected {dev}")
    return dev


def _rows(t: torch.Tensor, name: str):
    """Views [N, H*D] or [N, H, D] as (N, H, row stride, head stride); last dim must be dense."""
    if t.dim() == 2:
        if t.shape[1] % HEAD_SIZE != 0 or (t.shape[1] > 0 and t.stride(1) != 1):
            raise ValueError(f"{name}: expected [N, heads*{HEAD_SIZE}] with a dense last dim")
        return t.shape[0], t.shape[1] // HEAD_SIZE, t.stride(0), HEAD_SIZE
    if t.dim() == 3:
        if t.shape[2] != HEAD_SIZE or t.stride(2) != 1:
            raise ValueError(f"{name}: expected [N, heads, {HEAD_SIZE}] with a dense last dim")
        return t.shape[0], t.shape[1], t.stride(0), t.stride(1)
    raise ValueError(f"{name}: expected a 2-D or 3-D tensor")


def _pool(key_cache: torch.Tensor, value_cache: torch.Tensor):
    """Checks the pool layout of muxserve/flexstore/manager.py:456-468, returns (num_blocks, block_size)."""
    if key_cache.dim() != 4 or value_cache.dim() != 3:
        raise ValueError("key_cache must be [blocks, D/x, block, x] and value_cache [blocks, D, block]")
    if not key_cache.is_contiguous() or not value_cache.is_contiguous():
        raise ValueError("the KV pool tensors must be contiguous")
    nb, dx, bs, x = key_cache.shape
    if x * key_cache.element_size() != 16 or dx * x != HEAD_SIZE:
        raise ValueError(f"key_cache shape {tuple(key_cache.shape)} is not [blocks, {HEAD_SIZE}/x, block, x] with x = 16 bytes")
    if tuple(value_cache.shape) != (nb, HEAD_SIZE, bs):
        raise ValueError(f"value_cache shape {tuple(value_cache.shape)} does not match key_cache")
    if key_cache.dtype != value_cache.dtype:
        raise TypeError("key_cache and value_cache differ in dtype")
    return nb, bs


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes: int, device: torch.device) -> Optional[torch.Tensor]:
    """Scratch for partitioned (flash-decoding) launches, cached per (device, stream)."""
    if nbytes == 0:
        return None
    key = (device.index, _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reshape_and_cache(k: torch.Tensor, v: torch.Tensor, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Writes the new tokens' K/V rows into their pool slots.

    ``k``, ``v``: [T, H*128] or [T, H, 128] (views of a fused qkv tensor are fine);
    ``slot_mapping``: int64 [T, H], e.g. ``slot_mapping[:, layer, :]`` of the
    reference's [T, L, H] tensor (muxserve/flexserver/llm_runtime.py:301-302).
    Slot ``s`` is offset ``s % block_size`` of block ``s // block_size``
    (csrc/batch_scheduler.h:58-67); a negative slot skips the row.
    """
    _require_cuda(k=k, v=v, key_cache=key_cache, value_cache=value_cache, slot_mapping=slot_mapping)
    nb, bs = _pool(key_cache, value_cache)
    T, H, k_ts, k_hs = _rows(k, "k")
    Tv, Hv, v_ts, v_hs = _rows(v, "v")
    if (T, H) != (Tv, Hv):
        raise ValueError("k and v differ in shape")
    if k.dtype != key_cache.dtype or v.dtype != key_cache.dtype:
        raise TypeError("k/v dtype differs from the pool dtype")
    if slot_mapping.dtype != torch.int64:
        raise TypeError("slot_mapping must be int64")
    if slot_mapping.dim() == 1 and H == 1:
        slot_mapping = slot_mapping.unsqueeze(1)
    if slot_mapping.dim() != 2 or tuple(slot_mapping.shape) != (T, H):
        raise ValueError(f"slot_mapping must be [tokens, kv_heads] = [{T}, {H}], got {tuple(slot_mapping.shape)}")
    args = CacheWriteArgs(
        k=k.data_ptr(), v=v.data_ptr(), k_token_stride=k_ts, k_head_stride=k_hs,
        v_token_stride=v_ts, v_head_stride=v_hs,
        key_cache=key_cache.data_ptr(), value_cache=value_cache.data_ptr(), num_blocks=nb,
        slot_mapping=slot_mapping.data_ptr(),
        slot_token_stride=slot_mapping.stride(0), slot_head_stride=slot_mapping.stride(1),
        num_tokens=T, num_kv_heads=H, head_size=HEAD_SIZE, block_size=bs,
        dtype=_dtype_code(k, "k"), reserved=0)
    check(lib().mux_reshape_and_cache(C.byref(args), _stream()), "reshape_and_cache")
    global launch_count
    launch_count += 1 if T > 0 else 0


def paged_attention(out: torch.Tensor, q: torch.Tensor, key_cache: torch.Tensor,
                    value_cache: torch.Tensor, head_mapping: Optional[torch.Tensor], scale: float,
                    block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                    max_context_len: int, *, num_kv_heads: Optional[int] = None,
                    partition_size: int = 0, num_stages: int = 0, flags: int = 0,
                    seq_rows: Optional[torch.Tensor] = None, units: Optional[torch.Tensor] = None,
                    early_kv: bool = False, _new_kv=None, _rope=None) -> None:
    """Decode attention of one query token per sequence over the paged pool.

    ``q``/``out``: [S, Hq*128] or [S, Hq, 128].  ``block_tables``: int32
    [S, H, max_blocks] — one block list per (sequence, kv head), the per-layer
    slice of the reference's [L, S, H, max_blocks] tensor
    (muxserve/flexserver/llm_runtime.py:327) — or [S, max_blocks] when all kv
    heads share a list.  ``head_mapping``: int32 [Hq] kv head of each q head, or
    ``None`` for contiguous groups.  ``context_lens``: int32 [S], counting the
    token written by this step's ``reshape_and_cache``.  ``seq_rows`` (int32 [S], optional):
    sequence ``s`` uses row ``seq_rows[s]`` of ``block_tables`` (``device_tables.DeviceBlockTables``).
    ``units`` (``work_units(host context lengths, H, partition_size)``, optional): the real (item, partition) pairs,
    so that no CTA is launched for a partition a sequence does not have; needs the same explicit ``partition_size``.
    ``early_kv`` (``MUX_ATTN_EARLY_KV``): the caller states that neither the index tensors nor the KV blocks they name
    are written by the one or two kernels directly ahead of this call in the stream (true for a layer's
    ``decode_attention`` inside a decode step; NOT true right after ``reshape_and_cache`` of the same layer); the
    launch then stages its first KV blocks while those kernels drain.
    """
    if early_kv:
        flags |= _lib.MUX_ATTN_EARLY_KV
    _require_cuda(out=out, q=q, key_cache=key_cache, value_cache=value_cache, head_mapping=head_mapping,
                  block_tables=block_tables, context_lens=context_lens)
    nb, bs = _pool(key_cache, value_cache)
    if bs != block_size:
        raise ValueError(f"block_size {block_size} does not match the pool's {bs}")
    S, Hq, q_ss, q_hs = _rows(q, "q")
    So, Hqo, o_ss, o_hs = _rows(out, "out")
    if (S, Hq) != (So, Hqo):
        raise ValueError("q and out differ in shape")
    if q.dtype != key_cache.dtype or out.dtype != key_cache.dtype:
        raise TypeError("q/out dtype differs from the pool dtype")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise TypeError("block_tables and context_lens must be int32")
    if context_lens.dim() != 1 or context_lens.shape[0] != S or not context_lens.is_contiguous():
        raise ValueError("context_lens must be a contiguous [num_seqs] tensor")
    if block_tables.dim() == 3:
        if block_tables.stride(2) != 1 and block_tables.shape[2] > 1:
            raise ValueError("block_tables must be dense along the block dimension")
        H = block_tables.shape[1]
        bt_ss, bt_hs = block_tables.stride(0), block_tables.stride(1)
    elif block_tables.dim() == 2:
        if block_tables.stride(1) != 1 and block_tables.shape[1] > 1:
            raise ValueError("block_tables must be dense along the block dimension")
        H = num_kv_heads if num_kv_heads is not None else Hq
        bt_ss, bt_hs = block_tables.stride(0), 0
    else:
        raise ValueError("block_tables must be [S, H, max_blocks] or [S, max_blocks]")
    if num_kv_heads is not None and num_kv_heads != H:
        raise ValueError("num_kv_heads does not match block_tables")
    sr_ptr = None
    if seq_rows is not None:
        _require_cuda(seq_rows=seq_rows)
        if seq_rows.dtype != torch.int32 or seq_rows.dim() != 1 or seq_rows.shape[0] != S or not seq_rows.is_contiguous():
            raise ValueError("seq_rows must be a contiguous int32 [num_seqs] tensor")
        sr_ptr = seq_rows.data_ptr()
    elif block_tables.shape[0] != S:
        raise ValueError("block_tables and q differ in the number of sequences")
    if block_tables.shape[-1] * block_size < max_context_len:
        raise ValueError("block_tables has fewer blocks per sequence than max_context_len needs")
    hm_ptr = None
    if head_mapping is not None:
        if head_mapping.dtype != torch.int32 or head_mapping.numel() != Hq or not head_mapping.is_contiguous():
            raise ValueError("head_mapping must be a contiguous int32 [num_q_heads] tensor")
        hm_ptr = head_mapping.data_ptr()
    args = AttnArgs(
        out=out.data_ptr(), q=q.data_ptr(), q_seq_stride=q_ss, q_head_stride=q_hs,
        out_seq_stride=o_ss, out_head_stride=o_hs,
        key_cache=key_cache.data_ptr(), value_cache=value_cache.data_ptr(), num_blocks=nb,
        head_mapping=hm_ptr, block_tables=block_tables.data_ptr(),
        bt_seq_stride=bt_ss, bt_head_stride=bt_hs, context_lens=context_lens.data_ptr(), seq_rows=sr_ptr,
        scale=float(scale), num_seqs=S, num_q_heads=Hq, num_kv_heads=H, head_size=HEAD_SIZE,
        block_size=block_size, max_context_len=int(max_context_len), dtype=_dtype_code(q, "q"),
        partition_size=partition_size, num_stages=num_stages, flags=flags, num_units=0, units=None)
    if units is not None:
        _require_cuda(units=units)
        if units.dtype != torch.int32 or units.dim() != 1 or not units.is_contiguous() or partition_size <= 0:
            raise ValueError("units must be a contiguous int32 vector and needs an explicit partition_size")
        args.num_units, args.units = units.shape[0], units.data_ptr()
    L = lib()
    need = L.mux_paged_attention_workspace_size(C.byref(args))
    ws = _workspace(need, q.device)
    if _new_kv is None:
        check(L.mux_paged_attention(C.byref(args), ws.data_ptr() if ws is not None else None,
                                    ws.numel() if ws is not None else 0, _stream()), "paged_attention")
    else:
        k, v = _new_kv
        _require_cuda(k=k, v=v)
        if bt_hs == 0 and H > 1:
            raise ValueError("decode_attention appends one row per (sequence, kv head): every kv head needs its own "
                             "block list ([S, H, max_blocks] block_tables)")
        Tk, Hk, k_ss, k_hs = _rows(k, "k")
        Tv, Hv, v_ss, v_hs = _rows(v, "v")
        NT = Tk // S if S > 0 and Tk % S == 0 else 0
        if NT < 1 or NT > MAX_FUSED_NEW_TOKENS or (Tk, Hk) != (S * NT, H) or (Tv, Hv) != (Tk, H):
            raise ValueError(f"k and v must hold 1..{MAX_FUSED_NEW_TOKENS} new rows per (sequence, kv head), token-major "
                             f"within a sequence: [{S} * new_tokens, {H}, {HEAD_SIZE}]")
        if k.dtype != key_cache.dtype or v.dtype != key_cache.dtype:
            raise TypeError("k/v dtype differs from the pool dtype")
        rope_ptr, rope_len = _rope_cache(_rope, q)
        dargs = _lib.DecodeArgs(attn=args, k=k.data_ptr(), v=v.data_ptr(), k_seq_stride=k_ss, k_head_stride=k_hs,
                                v_seq_stride=v_ss, v_head_stride=v_hs, cos_sin_cache=rope_ptr, max_position=rope_len,
                                new_tokens=NT, reserved=0)
        check(L.mux_decode_attention(C.byref(dargs), ws.data_ptr() if ws is not None else None,
                                     ws.numel() if ws is not None else 0, _stream()), "decode_attention")
    global launch_count
    launch_count += 0 if S == 0 else (2 if need > 0 else 1)


def make_cos_sin_cache(max_position: int, base: float = 10000.0, dtype: torch.dtype = torch.float16,
                       device="cuda") -> torch.Tensor:
    """Rotary cache [max_position, 128] in the tensor dtype: 64 cosines then 64 sines of
    position * base^(-2i/128) (rope_theta and max_position_embeddings of llama.py:138-147)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, HEAD_SIZE, 2, dtype=torch.float32) / HEAD_SIZE))
    freqs = torch.outer(torch.arange(max_position, dtype=torch.float32), inv_freq)
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(dtype).to(device).contiguous()


def _rope_cache(cache: Optional[torch.Tensor], like: torch.Tensor):
    if cache is None:
        return None, 0
    if (not cache.is_cuda or cache.dim() != 2 or cache.shape[1] != HEAD_SIZE or not cache.is_contiguous()
            or cache.dtype != like.dtype):
        raise ValueError(f"cos_sin_cache must be a contiguous CUDA [max_position, {HEAD_SIZE}] tensor of the q dtype")
    return cache.data_ptr(), cache.shape[0]


def rotary_embedding(positions: torch.Tensor, q: Optional[torch.Tensor], k: Optional[torch.Tensor],
                     cos_sin_cache: torch.Tensor) -> None:
    """In-place rotary embedding (GPT-NeoX pairing, rotary dimension 128) of ``q`` [T, Hq(*128)] and ``k``
    [T, H(*128)] at ``positions`` (int64 [T]) — what PagedAttentionWithRoPE does before the cache write."""
    ref = q if q is not None else k
    _require_cuda(positions=positions, q=q, k=k, cos_sin_cache=cos_sin_cache)
    rope_ptr, rope_len = _rope_cache(cos_sin_cache, ref)
    if positions.dtype != torch.int64 or positions.dim() != 1 or not positions.is_contiguous():
        raise TypeError("positions must be a contiguous int64 [tokens] tensor")
    T = positions.shape[0]
    Tq, Hq, q_ts, q_hs = _rows(q, "q") if q is not None else (T, 0, 0, 0)
    Tk, Hk, k_ts, k_hs = _rows(k, "k") if k is not None else (T, 0, 0, 0)
    if Tq != T or Tk != T:
        raise ValueError("positions, q and k differ in the number of tokens")
    args = _lib.RotaryArgs(q=q.data_ptr() if q is not None else None, k=k.data_ptr() if k is not None else None,
                           q_token_stride=q_ts, q_head_stride=q_hs, k_token_stride=k_ts, k_head_stride=k_hs,
                           positions=positions.data_ptr(), cos_sin_cache=rope_ptr, max_position=rope_len,
                           num_tokens=T, num_q_heads=Hq, num_kv_heads=Hk, head_size=HEAD_SIZE,
                           dtype=_dtype_code(ref, "q/k"), reserved=0)
    check(lib().mux_rotary_embedding(C.byref(args), _stream()), "rotary_embedding")
    global launch_count
    launch_count += 1 if T > 0 and Hq + Hk > 0 else 0


def work_units(item_context_lens, partition_size: int, device=None, num_kv_heads: Optional[int] = None):
    """Work list for the ``units=`` argument of the attention ops, from context lengths the HOST holds.

    ``item_context_lens``: one length per (sequence, kv head) item — or one per sequence together with
    ``num_kv_heads`` (item = sequence * num_kv_heads + kv head).  Returns int32 ``item | partition << 24`` for every
    real (item, partition) pair, fullest partitions first (a numpy array, or a tensor on ``device``).  An item with
    an empty context gets its partition 0 too: that CTA writes the zeros the launch without a list would write."""
    import numpy as np
    ctx = np.asarray(item_context_lens, dtype=np.int64).reshape(-1)
    if num_kv_heads is not None:
        ctx = np.repeat(ctx, num_kv_heads)
    if partition_size <= 0:
        raise ValueError("the work list is built for an explicit partition size")
    nparts = np.maximum(1, (np.maximum(ctx, 0) + partition_size - 1) // partition_size)
    if ctx.size >= 1 << 24 or (nparts.size and int(nparts.max()) > 128):
        raise ValueError("too many items or partitions for a packed work list")
    item = np.repeat(np.arange(ctx.size, dtype=np.int64), nparts)
    first = np.cumsum(nparts) - nparts
    part = np.arange(item.size, dtype=np.int64) - np.repeat(first, nparts)
    tokens = np.minimum(partition_size, np.maximum(ctx[item], 0) - part * partition_size)
    order = np.argsort(-tokens, kind="stable")
    packed = (item[order] | (part[order] << 24)).astype(np.uint32).view(np.int32).copy()
    return packed if device is None else torch.from_numpy(packed).to(device)


def suggest_launch(item_context_lens, group: int, device=None, num_kv_heads: Optional[int] = None):
    """(partition_size, num_stages) for a launch with a work list, from context lengths the HOST holds (one per
    (sequence, kv head) item, or one per sequence together with ``num_kv_heads``).

    Encodes what sweeps on B200 showed (148 SMs, six resident CTAs each at the default ring = 888 CTA places; one
    CTA alone streams only ~25 GB/s, so a launch is fast when its work covers the places and no unit is much longer
    than the rest):
    * 512-token partitions unless the launch is much larger or much smaller than the places;
    * one or two q heads per kv head and more than ~2 units per place at 512: the longest partition that still
      gives every place a unit (no split at all for big batches: no partial results, no merge kernel);
    * fewer than ~0.4 units per place at 512: the longest shorter partition that covers two thirds of the places;
    * a launch that fills the places about once takes a 12-deep ring (four fuller CTAs per SM);
    * grouped heads keep 512 and the default ring (their logits rows take shared memory in proportion)."""
    import numpy as np
    ctx = np.asarray(item_context_lens, dtype=np.int64).reshape(-1)
    if num_kv_heads is not None:
        ctx = np.repeat(ctx, num_kv_heads)
    if group > 2 or ctx.size == 0:
        return 512, 0
    sms = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    places = 6 * sms
    units = lambda psize: int(((np.maximum(ctx, 1) + psize - 1) // psize).sum())
    top = 128
    while top < min(4096, int(ctx.max())):
        top *= 2
    psize = min(512, top)
    if units(512) > 2.2 * places:
        for cand in (4096, 2048, 1024):
            if cand <= top and units(cand) >= places:
                psize = cand
                break
    elif units(512) < 0.4 * places:
        psize = 128
        for cand in (256,):
            if units(cand) >= 0.68 * places:
                psize = cand
    stages = 12 if psize >= 512 and units(psize) <= 1.2 * places else 0
    return psize, stages


def suggest_partition_size(num_items: int, group: int, device=None) -> int:
    """Partition size when only the item count is known (see ``suggest_launch`` for the rule with the lengths)."""
    sms = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    return 2048 if group <= 2 and num_items >= 2 * 6 * sms else 512


def decode_attention(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     key_cache: torch.Tensor, value_cache: torch.Tensor, head_mapping: Optional[torch.Tensor],
                     scale: float, block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                     max_context_len: int, *, cos_sin_cache: Optional[torch.Tensor] = None, **kw) -> None:
    """``reshape_and_cache`` + ``paged_attention`` of one layer's decode step in one launch.

    ``k``, ``v``: [S, H*128] or [S, H, 128], the new token of every sequence.  Row (s, h) is
    appended at position ``context_lens[s] - 1`` of block list ``block_tables[s, h]`` — the slot
    the reference's ``slot_mapping`` names for a decode step (csrc/batch_scheduler.h:58-67) — and
    attention runs over all ``context_lens[s]`` tokens.  Results equal the two separate ops bit for bit.
    ``k``, ``v`` may also hold n <= 16 new rows per sequence, [S*n, H(*128)] token-major within a sequence: they go
    to positions ``context_lens[s] - n .. context_lens[s] - 1`` (the context length counts them all).
    With ``cos_sin_cache`` the query and the new key are first rotated at position ``context_lens[s] - 1``
    (neither ``q`` nor ``k`` is modified), as ``rotary_embedding`` would.
    """
    paged_attention(out, q, key_cache, value_cache, head_mapping, scale, block_tables, context_lens,
                    block_size, max_context_len, _new_kv=(k, v), _rope=cos_sin_cache, **kw)


def paged_attention_mixed(out: torch.Tensor, q: torch.Tensor, key_cache: torch.Tensor,
                          value_cache: torch.Tensor, block_tables: torch.Tensor,
                          item_context_len: torch.Tensor, item_q_row: torch.Tensor,
                          item_group: torch.Tensor, item_scale: torch.Tensor, block_size: int,
                          max_context_len: int, max_group: int, *, partition_size: int = 0,
                          num_stages: int = 0, flags: int = 0, new_k: Optional[torch.Tensor] = None,
                          new_v: Optional[torch.Tensor] = None, cos_sin_cache: Optional[torch.Tensor] = None,
                          units: Optional[torch.Tensor] = None, early_kv: bool = False) -> None:
    """One launch for the decode batches of several models sharing the pool.

    Item ``i`` is one (sequence, kv head) of some model: q rows
    ``item_q_row[i] .. + item_group[i]`` of the packed ``q``/``out`` [rows, 128]
    attend over block list ``block_tables[i]`` with ``item_context_len[i]`` tokens
    and softmax scale ``item_scale[i]``.  ``muxserve_b200.mixed`` builds these
    arrays from per-model batches.  With ``new_k`` / ``new_v`` ([items, 128], one new row per
    item) the call is the whole decode step: every row is first appended at position
    ``item_context_len[i] - 1`` of its block list, as ``decode_attention`` does.
    ``units`` (``MixedPlan.units(layer, partition_size)``, int32) lists the real (item, partition) pairs so that no
    CTA is launched for a partition an item does not have; ``partition_size`` must then be the one the list was built for.
    ``early_kv``: as in ``paged_attention``.
    """
    if early_kv:
        flags |= _lib.MUX_ATTN_EARLY_KV
    _require_cuda(out=out, q=q, key_cache=key_cache, value_cache=value_cache, block_tables=block_tables,
                  item_context_len=item_context_len, item_q_row=item_q_row, item_group=item_group,
                  item_scale=item_scale)
    nb, bs = _pool(key_cache, value_cache)
    if bs != block_size:
        raise ValueError(f"block_size {block_size} does not match the pool's {bs}")
    if q.dim() != 2 or q.shape[1] != HEAD_SIZE or q.stride(1) != 1 or out.shape != q.shape or out.stride(1) != 1:
        raise ValueError(f"q and out must be packed [rows, {HEAD_SIZE}] tensors of one shape")
    if q.dtype != key_cache.dtype or out.dtype != key_cache.dtype:
        raise TypeError("q/out dtype differs from the pool dtype")
    n = block_tables.shape[0]
    if block_tables.dim() != 2 or block_tables.dtype != torch.int32 or (block_tables.shape[1] > 1 and block_tables.stride(1) != 1):
        raise ValueError("block_tables must be int32 [items, max_blocks], dense along blocks")
    for name, t, dt in (("item_context_len", item_context_len, torch.int32), ("item_q_row", item_q_row, torch.int32),
                        ("item_group", item_group, torch.int32), ("item_scale", item_scale, torch.float32)):
        if t.dtype != dt or t.dim() != 1 or t.shape[0] != n or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous {dt} [items] tensor")
    if block_tables.shape[1] * block_size < max_context_len:
        raise ValueError("block_tables has fewer blocks per item than max_context_len needs")
    args = AttnMixedArgs(
        out=out.data_ptr(), q=q.data_ptr(), q_row_stride=q.stride(0), out_row_stride=out.stride(0),
        key_cache=key_cache.data_ptr(), value_cache=value_cache.data_ptr(), num_blocks=nb,
        block_tables=block_tables.data_ptr(), bt_item_stride=block_tables.stride(0),
        item_context_len=item_context_len.data_ptr(), item_q_row=item_q_row.data_ptr(),
        item_group=item_group.data_ptr(), item_scale=item_scale.data_ptr(),
        num_items=n, max_group=max_group, head_size=HEAD_SIZE, block_size=block_size,
        max_context_len=int(max_context_len), dtype=_dtype_code(q, "q"),
        partition_size=partition_size, num_stages=num_stages, flags=flags, num_units=0, units=None)
    if units is not None:
        _require_cuda(units=units)
        if units.dtype != torch.int32 or units.dim() != 1 or not units.is_contiguous() or partition_size <= 0:
            raise ValueError("units must be a contiguous int32 vector and needs an explicit partition_size")
        args.num_units, args.units = units.shape[0], units.data_ptr()
    L = lib()
    need = L.mux_paged_attention_mixed_workspace_size(C.byref(args))
    ws = _workspace(need, q.device)
    if new_k is None and new_v is None:
        check(L.mux_paged_attention_mixed(C.byref(args), ws.data_ptr() if ws is not None else None,
                                          ws.numel() if ws is not None else 0, _stream()),
              "paged_attention_mixed")
    else:
        _require_cuda(new_k=new_k, new_v=new_v)
        NT = new_k.shape[0] // n if n > 0 and new_k.dim() == 2 and new_k.shape[0] % n == 0 else 0
        for name, t in (("new_k", new_k), ("new_v", new_v)):
            if (NT < 1 or NT > MAX_FUSED_NEW_TOKENS or t.dim() != 2 or tuple(t.shape) != (n * NT, HEAD_SIZE)
                    or t.stride(1) != 1 or t.dtype != q.dtype):
                raise ValueError(f"{name} must be [{n} * new_tokens, {HEAD_SIZE}] of the pool dtype with a dense last dim")
        rope_ptr, rope_len = _rope_cache(cos_sin_cache, q)
        dargs = _lib.DecodeMixedArgs(attn=args, k=new_k.data_ptr(), v=new_v.data_ptr(),
                                     k_row_stride=new_k.stride(0), v_row_stride=new_v.stride(0),
                                     cos_sin_cache=rope_ptr, max_position=rope_len, new_tokens=NT, reserved=0)
        check(L.mux_decode_attention_mixed(C.byref(dargs), ws.data_ptr() if ws is not None else None,
                                           ws.numel() if ws is not None else 0, _stream()),
              "decode_attention_mixed")
    global launch_count
    launch_count += 0 if n == 0 else (2 if need > 0 else 1)


def cu_seqlens_from_prompt_lens(prompt_lens, device) -> torch.Tensor:
    """int32 [len(prompt_lens) + 1] prefix sums of ``prompt_lens`` (``InputMetadata.prompt_lens``) on ``device``."""
    cu = [0]
    for n in prompt_lens:
        cu.append(cu[-1] + int(n))
    return torch.tensor(cu, dtype=torch.int32, device=device)


def prefill_work_units(prompt_lens, num_q_heads: int, device=None):
    """Work list for ``prefill_attention(..., units=)`` from the prompt lengths the HOST holds: int32 [U, 2] rows
    ``(prompt, q head | query tile << 16)``, one per 128-row query tile of every (prompt, q head); prompts in order
    of decreasing length, the tiles of one (prompt, head) together (they share their K/V in L2), last tile first."""
    import numpy as np
    lens = np.asarray(prompt_lens, dtype=np.int64).reshape(-1)
    if num_q_heads >= 1 << 16 or (lens.size and (int(lens.max()) + 127) // 128 >= 1 << 15):
        raise ValueError("too many heads or tiles for a packed work list")
    rows = []
    for s in np.argsort(-lens, kind="stable"):
        tiles = (int(lens[s]) + 127) // 128
        if tiles == 0:
            continue
        qt = np.arange(tiles - 1, -1, -1, dtype=np.int64)
        h = np.arange(num_q_heads, dtype=np.int64)
        hq = (h[:, None] | (qt[None, :] << 16)).reshape(-1)
        rows.append(np.stack([np.full(hq.size, s, dtype=np.int64), hq], axis=1))
    packed = (np.concatenate(rows) if rows else np.zeros((0, 2), dtype=np.int64)).astype(np.int32)
    return packed if device is None else torch.from_numpy(packed).to(device)


def prefill_attention(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      cu_seqlens: torch.Tensor, max_prompt_len: int, scale: float,
                      key_cache: Optional[torch.Tensor] = None, value_cache: Optional[torch.Tensor] = None,
                      slot_mapping: Optional[torch.Tensor] = None,
                      block_tables: Optional[torch.Tensor] = None, units: Optional[torch.Tensor] = None) -> None:
    """Causal self-attention of every prompt over its own tokens (the prompt branch of PagedAttentionWithRoPE).

    ``q``/``out`` [T, Hq(*128)], ``k``/``v`` [T, H(*128)] hold the rows of all prompts back to back;
    ``cu_seqlens`` int32 [S + 1] (device) are the row offsets; ``max_prompt_len`` bounds every prompt length.
    With ``key_cache``/``value_cache``/``slot_mapping`` (int64 [T, H], e.g. ``slot_mapping[:, layer, :]``) the same
    launch also writes every K/V row to its pool slot, bit for bit what ``reshape_and_cache`` would write.
    ``block_tables`` (int32 [S, H, max_blocks], this layer's lists as the decode ops take them) may stand in for
    ``slot_mapping``: token t of a prompt goes to offset ``t % block_size`` of block ``t // block_size`` of its list.
    ``units`` (``prefill_work_units(prompt_lens, Hq, device)``, int32 [U, 2]): the real (prompt, q head, query tile)
    triples, longest prompts first, so that no CTA is launched for a tile a prompt does not have."""
    _require_cuda(out=out, q=q, k=k, v=v, cu_seqlens=cu_seqlens, key_cache=key_cache, value_cache=value_cache,
                  slot_mapping=slot_mapping, block_tables=block_tables)
    if cu_seqlens.dtype != torch.int32 or cu_seqlens.dim() != 1 or not cu_seqlens.is_contiguous():
        raise TypeError("cu_seqlens must be a contiguous int32 [num_seqs + 1] tensor")
    code = _dtype_code(q, "q")
    if out.dtype != q.dtype or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("out, q, k and v must have one dtype")
    T, Hq, q_ss, q_hs = _rows(q, "q")
    To, Ho, o_ss, o_hs = _rows(out, "out")
    Tk, Hk, k_ss, k_hs = _rows(k, "k")
    Tv, Hv, v_ss, v_hs = _rows(v, "v")
    if (To, Ho) != (T, Hq) or Tk != T or Tv != T or Hv != Hk:
        raise ValueError("out/q/k/v shapes do not agree")
    S = cu_seqlens.shape[0] - 1
    if S < 0:
        raise ValueError("cu_seqlens needs at least one entry")
    pool = dict(block_size=0, key_cache=None, value_cache=None, slot_mapping=None, slot_token_stride=0,
                slot_head_stride=0, num_blocks=0, block_tables=None, bt_seq_stride=0, bt_head_stride=0,
                max_blocks_per_seq=0, num_units=0, units=None)
    if key_cache is not None or value_cache is not None or slot_mapping is not None or block_tables is not None:
        if key_cache is None or value_cache is None or (slot_mapping is None) == (block_tables is None):
            raise ValueError("the cache write needs key_cache, value_cache and ONE of slot_mapping / block_tables")
        nb, bs = _pool(key_cache, value_cache)
        if key_cache.dtype != q.dtype:
            raise TypeError("k/v dtype differs from the pool dtype")
        pool.update(block_size=bs, key_cache=key_cache.data_ptr(), value_cache=value_cache.data_ptr(), num_blocks=nb)
        if slot_mapping is not None:
            if slot_mapping.dtype != torch.int64 or tuple(slot_mapping.shape) != (T, Hk):
                raise ValueError(f"slot_mapping must be int64 [tokens, kv_heads] = [{T}, {Hk}]")
            pool.update(slot_mapping=slot_mapping.data_ptr(), slot_token_stride=slot_mapping.stride(0),
                        slot_head_stride=slot_mapping.stride(1))
        else:
            if (block_tables.dtype != torch.int32 or block_tables.dim() != 3 or block_tables.shape[:2] != (S, Hk)
                    or (block_tables.shape[2] > 1 and block_tables.stride(2) != 1)):
                raise ValueError(f"block_tables must be int32 [num_seqs, kv_heads, max_blocks] = [{S}, {Hk}, *]")
            pool.update(block_tables=block_tables.data_ptr(), bt_seq_stride=block_tables.stride(0),
                        bt_head_stride=block_tables.stride(1), max_blocks_per_seq=block_tables.shape[2])
    args = _lib.PrefillArgs(out=out.data_ptr(), q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(),
                            out_seq_stride=o_ss, out_head_stride=o_hs, q_seq_stride=q_ss, q_head_stride=q_hs,
                            k_seq_stride=k_ss, k_head_stride=k_hs, v_seq_stride=v_ss, v_head_stride=v_hs,
                            cu_seqlens=cu_seqlens.data_ptr(), scale=float(scale), num_seqs=S, total_tokens=T,
                            max_prompt_len=int(max_prompt_len), num_q_heads=Hq, num_kv_heads=Hk,
                            head_size=HEAD_SIZE, dtype=code, **pool)
    if units is not None:
        _require_cuda(units=units)
        if units.dtype != torch.int32 or units.dim() != 2 or units.shape[1] != 2 or not units.is_contiguous():
            raise ValueError("units must be a contiguous int32 [U, 2] tensor")
        args.num_units, args.units = units.shape[0], units.data_ptr()
    check(lib().mux_prefill_attention(C.byref(args), _stream()), "prefill_attention")
    global launch_count
    launch_count += 1 if S > 0 and T > 0 and max_prompt_len > 0 else 0


def device_status() -> int:
    """Reads and clears the MUX_DEV_* status bits of the current device (synchronises the stream)."""
    return check(lib().mux_device_status(_stream()), "device_status")
