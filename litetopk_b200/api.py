"""Python-facing operators of the LiteDSA sparse-attention hot path on B200.

Two layers, both thin wrappers over the C ABI (include/litedsa_b200.h):

* ``*_out`` functions take exactly the argument lists of the reference's TVM-FFI
  operators (kernels/b200/dsa/litedsa_jit_binding.cu:7-17) -- destination passing,
  caller-owned outputs, nothing allocated, asynchronous on the current stream.
* ``union_qm`` / ``masked_mla_fp8`` are the allocate-and-return forms.

Dtypes, devices and contiguity are checked here (the reference checks shapes only and
casts pointers blindly, litedsa.cu:70-72, 111-124); shape rules are checked again in C.
There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(t: torch.Tensor, name: str, dtype, ndim: Optional[int] = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    dts = dtype if isinstance(dtype, (tuple, list)) else (dtype,)
    if t.dtype not in dts:
        raise TypeError(f"{name} must have dtype {dts}, got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must be {ndim}-D, got shape {tuple(t.shape)}")


def _mask_dtype_ok(t: torch.Tensor) -> bool:
    return t.dtype in (torch.int32, torch.uint32)


# --------------------------------------------------------------------------- union
def union_qm_out(topk_indices: torch.Tensor, u_phys: torch.Tensor, counts: torch.Tensor,
                 memb_qm: torch.Tensor, req_pg: Optional[torch.Tensor],
                 block_table: Optional[torch.Tensor], block_size: int, seq_space: int,
                 *, fill_tail: bool = False) -> None:
    """Reference argument order (kernels/b200/dsa/litedsa.cu:31-33).

    topk_indices [T,k] i32; u_phys [ng,cap] i32; counts [ng] i32; memb_qm [ng,G,cap/32]
    u32 bits (int32 storage accepted); req_pg [ng] i32 and block_table [nreq,nblk] i32, or
    both None for an identity table.  Entries beyond the live prefixes are left untouched
    unless ``fill_tail``.
    """
    _need(topk_indices, "topk_indices", torch.int32, 2)
    _need(u_phys, "u_phys", torch.int32, 2)
    _need(counts, "counts", torch.int32, 1)
    _need(memb_qm, "memb_qm", (torch.int32, torch.uint32), 3)
    for name, t in (("topk_indices", topk_indices), ("u_phys", u_phys), ("counts", counts),
                    ("memb_qm", memb_qm)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    T, k = topk_indices.shape
    ng, cap = u_phys.shape
    G = memb_qm.shape[1]
    if memb_qm.shape[0] != ng or memb_qm.shape[2] * 32 != cap:
        raise ValueError("memb_qm must be [ng, G, cap/32]")
    if counts.shape[0] != ng:
        raise ValueError("counts must be [ng]")
    bt_rows = bt_blocks = 0
    if (req_pg is None) != (block_table is None):
        raise ValueError("req_pg and block_table must be given together")
    if block_table is not None:
        _need(req_pg, "req_pg", torch.int32, 1)
        _need(block_table, "block_table", torch.int32, 2)
        if not (req_pg.is_contiguous() and block_table.is_contiguous()):
            raise ValueError("req_pg / block_table must be contiguous")
        if req_pg.shape[0] != ng:
            raise ValueError("req_pg must be [ng]")
        bt_rows, bt_blocks = block_table.shape
    with torch.cuda.device(topk_indices.device):
        rc = _lib.lib().litedsa_union_qm(
            _ptr(topk_indices), _ptr(u_phys), _ptr(counts), _ptr(memb_qm), _ptr(req_pg),
            _ptr(block_table), T, k, ng, cap, G, bt_rows, bt_blocks, int(block_size),
            int(seq_space), 1 if fill_tail else 0, _stream(topk_indices))
    check(rc, "union_qm")


def union_qm(topk_idx: torch.Tensor, tokens_per_tile: int, *, seq_space: Optional[int] = None,
             return_counts: bool = False):
    """Deduplicated per-tile KV index list + query-major membership bitmask.

    topk_idx [T,k] int32 (-1 = padding).  Returns ``(union_idx [ng, G*k] int32, mask
    [ng, G, G*k/32] int32 holding u32 bit words)`` and, with ``return_counts``, also
    ``counts [ng] int32``.  union_idx is ascending with -1 beyond each tile's count; mask
    words beyond it are zero.  ``seq_space`` bounds valid positions (default: 2^20, the
    operator's maximum).
    """
    _need(topk_idx, "topk_idx", torch.int32, 2)
    T, k = topk_idx.shape
    G = int(tokens_per_tile)
    if G <= 0 or T % G != 0:
        raise ValueError("number of tokens must be a multiple of tokens_per_tile")
    ng, cap = T // G, G * k
    dev = topk_idx.device
    u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
    mask = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
    space = 1 << 20 if seq_space is None else ((int(seq_space) + 1023) // 1024) * 1024
    union_qm_out(topk_idx.contiguous(), u, cnt, mask, None, None, 1, space, fill_tail=True)
    return (u, mask, cnt) if return_counts else (u, mask)


# --------------------------------------------------------------------------- FP8 attention
def masked_mla_fp8_out(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                       out_scale: float, topk_length: Optional[torch.Tensor],
                       memb_qm: Optional[torch.Tensor], h_per_q: int, out: torch.Tensor,
                       max_logits: Optional[torch.Tensor], lse: torch.Tensor,
                       *, peer_outs=None, attn_sink: Optional[torch.Tensor] = None,
                       topk_length_per_q: Optional[torch.Tensor] = None,
                       q_group_div: int = 1, in_place_heads: bool = False) -> None:
    """Reference argument order (kernels/b200/dsa/litedsa.cu:77-80).

    q [ng,128,576] e4m3 (uint8 storage accepted); kv [s_kv,1,576] or [s_kv,576] e4m3, row
    pitch = kv.stride(0); indices [ng,1,topk] or [ng,topk] i32 physical slots; topk_length
    [ng] i32 (None: every tile uses topk); memb_qm [ng,G,topk/32] u32 bits; out
    [ng,128,512] bf16; max_logits [ng,128] f32 or None; lse [ng,128] f32.
    logits = sm_scale * (q . k); out = out_scale * softmax(logits) @ kv[:, :512].

    Keyword extras.  ``peer_outs`` (sharded multi-GPU runs): up to seven peer-mapped device
    addresses (ints) of [ng,128,512] bf16 buffers on other GPUs that receive a copy of every
    output box from the kernel's epilogue (see :mod:`litetopk_b200.dist`).  The optional modes
    of the reference kernel's parameter block (litedsa_attention_sm100.cuh:1340-1393):
    ``attn_sink`` [128] f32 per packed row joins the output normaliser; ``topk_length_per_q``
    [ng,G] i32 bounds each token to a causal prefix of the union ranks (memb_qm may then be
    None); ``q_group_div`` consecutive tiles share one Q tile (q is [ng/q_group_div,128,576]).

    ``in_place_heads`` (zero-copy for tensor-parallel callers): q is the model's own
    ``[T, H_padded, 576]`` tensor and out its ``[T, H_padded, 512]`` tensor, of which only the
    first ``h_per_q`` head slots of every token are read / written (G = 128 // h_per_q
    consecutive tokens form a tile); any token / head strides with unit inner stride and
    16-byte-multiple pitches.  This removes the pack and unpack copies the reference's packed
    path performs around its kernel (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:12-22).
    lse / max_logits stay packed ``[ng,128]``.
    """
    f8 = (torch.float8_e4m3fn, torch.uint8)
    _need(q, "q", f8, 3)
    _need(kv, "kv", f8)
    _need(indices, "indices", torch.int32)
    _need(out, "out", torch.bfloat16, 3)
    _need(lse, "lse", torch.float32)
    if kv.dim() == 3:
        if kv.shape[1] != 1:
            raise ValueError("kv must be [s_kv, 1, 576]")
        kv = kv[:, 0]
    if indices.dim() == 3:
        if indices.shape[1] != 1:
            raise ValueError("indices must be [ng, 1, topk]")
        indices = indices[:, 0]
    ng = indices.shape[0]
    q_group_div = int(q_group_div)
    G = 128 // int(h_per_q)
    q_strides = out_strides = (0, 0)
    if in_place_heads:
        if q_group_div < 1 or ng % q_group_div or q.dim() != 3 or q.shape[0] != ng // q_group_div * G \
                or q.shape[1] < h_per_q or q.shape[2] != 576 or kv.shape[1] != 576:
            raise ValueError("in_place_heads: q must be [ng*G/q_group_div, H_padded >= h_per_q, 576]")
        if tuple(out.shape[:1]) != (ng * G,) or out.shape[1] < h_per_q or out.shape[2] != 512:
            raise ValueError("in_place_heads: out must be [ng*G, H_padded >= h_per_q, 512]")
        if q.stride(2) != 1 or out.stride(2) != 1 or kv.stride(1) != 1 or indices.stride(1) != 1:
            raise ValueError("q / out / kv / indices need unit inner stride")
        q_strides = (q.stride(0), q.stride(1))
        out_strides = (out.stride(0), out.stride(1))
    else:
        if q_group_div < 1 or ng % q_group_div or tuple(q.shape) != (ng // q_group_div, 128, 576) \
                or kv.shape[1] != 576:
            raise ValueError("q must be [ng/q_group_div,128,576] and kv [s_kv,(1,)576]")
        if q.stride(2) != 1 or q.stride(1) * 128 != q.stride(0) or kv.stride(1) != 1 or indices.stride(1) != 1:
            raise ValueError("q rows must be evenly pitched; q/kv/indices need unit inner stride")
    topk = indices.shape[1]
    if memb_qm is None and topk_length_per_q is None:
        raise ValueError("memb_qm or topk_length_per_q is required")
    if memb_qm is not None:
        _need(memb_qm, "memb_qm", (torch.int32, torch.uint32))
        if memb_qm.numel() != ng * G * (topk // 32) or not memb_qm.is_contiguous():
            raise ValueError("memb_qm must be a contiguous [ng, G, topk/32]")
    if not in_place_heads and (tuple(out.shape) != (ng, 128, 512) or not out.is_contiguous()):
        raise ValueError("out must be a contiguous [ng,128,512]")
    if lse.numel() != ng * 128 or not lse.is_contiguous():
        raise ValueError("lse must be a contiguous [ng,128]")
    if topk_length is not None:
        _need(topk_length, "topk_length", torch.int32, 1)
        if topk_length.shape[0] != ng or not topk_length.is_contiguous():
            raise ValueError("topk_length must be a contiguous [ng]")
    if max_logits is not None:
        _need(max_logits, "max_logits", torch.float32)
        if max_logits.numel() != ng * 128 or not max_logits.is_contiguous():
            raise ValueError("max_logits must be a contiguous [ng,128]")
    if attn_sink is not None:
        _need(attn_sink, "attn_sink", torch.float32, 1)
        if attn_sink.shape[0] != 128 or not attn_sink.is_contiguous():
            raise ValueError("attn_sink must be a contiguous [128] (one value per packed row)")
    if topk_length_per_q is not None:
        _need(topk_length_per_q, "topk_length_per_q", torch.int32, 2)
        if tuple(topk_length_per_q.shape) != (ng, G) or not topk_length_per_q.is_contiguous():
            raise ValueError("topk_length_per_q must be a contiguous [ng, G]")
    extras = attn_sink is not None or topk_length_per_q is not None or q_group_div != 1 or in_place_heads
    q_row_stride = q.stride(1)
    with torch.cuda.device(q.device):
        if peer_outs:
            if extras:
                raise ValueError("peer_outs cannot be combined with attn_sink / topk_length_per_q / q_group_div")
            import ctypes
            ptrs = [_ptr(out)] + [int(a) for a in peer_outs]
            if len(ptrs) > 8:
                raise ValueError("at most 7 peer destinations")
            arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
            rc = _lib.lib().litedsa_masked_mla_fp8_multi(
                _ptr(q), _ptr(kv), _ptr(indices), float(sm_scale), float(out_scale),
                _ptr(topk_length), _ptr(memb_qm), int(h_per_q), arr, len(ptrs), _ptr(max_logits),
                _ptr(lse), ng, kv.shape[0], topk, q.stride(1), kv.stride(0), indices.stride(0),
                _stream(q))
        elif extras:
            rc = _lib.lib().litedsa_masked_mla_fp8_ex(
                _ptr(q), _ptr(kv), _ptr(indices), float(sm_scale), float(out_scale),
                _ptr(topk_length), _ptr(memb_qm), int(h_per_q), _ptr(out), _ptr(max_logits),
                _ptr(lse), ng, kv.shape[0], topk, q_row_stride, kv.stride(0), indices.stride(0),
                _ptr(attn_sink), _ptr(topk_length_per_q), q_group_div, q_strides[0], q_strides[1],
                out_strides[0], out_strides[1], _stream(q))
        else:
            rc = _lib.lib().litedsa_masked_mla_fp8(
                _ptr(q), _ptr(kv), _ptr(indices), float(sm_scale), float(out_scale),
                _ptr(topk_length), _ptr(memb_qm), int(h_per_q), _ptr(out), _ptr(max_logits),
                _ptr(lse), ng, kv.shape[0], topk, q.stride(1), kv.stride(0), indices.stride(0),
                _stream(q))
    check(rc, "masked_mla_fp8")


def _bf16_common(q, kv, indices, out, lse):
    _need(q, "q", torch.bfloat16, 3)
    _need(kv, "kv", torch.bfloat16)
    _need(indices, "indices", torch.int32)
    _need(out, "out", torch.bfloat16, 3)
    _need(lse, "lse", torch.float32)
    if kv.dim() == 3:
        if kv.shape[1] != 1:
            raise ValueError("kv must be [s_kv, 1, d]")
        kv = kv[:, 0]
    if indices.dim() == 3:
        if indices.shape[1] != 1:
            raise ValueError("indices must be [ng, 1, topk]")
        indices = indices[:, 0]
    ng, rows, d = q.shape
    if rows != 128 or d not in (512, 576) or kv.shape[1] != d:
        raise ValueError("q must be [ng,128,d] and kv [s_kv,(1,)d] with d = 512 or 576")
    if q.stride(2) != 1 or q.stride(1) * 128 != q.stride(0) or kv.stride(1) != 1 or indices.stride(1) != 1:
        raise ValueError("q rows must be evenly pitched; q/kv/indices need unit inner stride")
    if indices.shape[0] != ng:
        raise ValueError("indices rows must match q tiles")
    if tuple(out.shape) != (ng, 128, 512) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [ng,128,512]")
    if lse.numel() != ng * 128 or not lse.is_contiguous():
        raise ValueError("lse must be a contiguous [ng,128]")
    return kv, indices, ng, d


def _sink128(attn_sink):
    if attn_sink is None:
        return None
    _need(attn_sink, "attn_sink", torch.float32, 1)
    if attn_sink.shape[0] != 128 or not attn_sink.is_contiguous():
        raise ValueError("attn_sink must be a contiguous [128] (one value per packed row)")
    return attn_sink


def masked_mla_bf16_out(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                        topk_length: Optional[torch.Tensor], memb_qm: torch.Tensor, h_per_q: int,
                        out: torch.Tensor, max_logits: Optional[torch.Tensor], lse: torch.Tensor,
                        *, attn_sink: Optional[torch.Tensor] = None) -> None:
    """bf16 twin of :func:`masked_mla_fp8_out` (same argument order without ``out_scale``):
    q [ng,128,d] bf16, kv [s_kv,(1,)d] bf16 workspace (d = 576 or 512, V = first 512 dims),
    union list + query-major membership mask.  For caches with no single-scale e4m3 form."""
    kv, indices, ng, d = _bf16_common(q, kv, indices, out, lse)
    topk = indices.shape[1]
    G = 128 // int(h_per_q)
    _need(memb_qm, "memb_qm", (torch.int32, torch.uint32))
    if memb_qm.numel() != ng * G * (topk // 32) or not memb_qm.is_contiguous():
        raise ValueError("memb_qm must be a contiguous [ng, G, topk/32]")
    if topk_length is not None:
        _need(topk_length, "topk_length", torch.int32, 1)
        if topk_length.shape[0] != ng or not topk_length.is_contiguous():
            raise ValueError("topk_length must be a contiguous [ng]")
    if max_logits is not None:
        _need(max_logits, "max_logits", torch.float32)
        if max_logits.numel() != ng * 128 or not max_logits.is_contiguous():
            raise ValueError("max_logits must be a contiguous [ng,128]")
    with torch.cuda.device(q.device):
        rc = _lib.lib().litedsa_masked_mla_bf16(
            _ptr(q), _ptr(kv), _ptr(indices), float(sm_scale), _ptr(topk_length), _ptr(memb_qm),
            int(h_per_q), _ptr(out), _ptr(max_logits), _ptr(lse), ng, kv.shape[0], topk, d,
            q.stride(1), kv.stride(0), indices.stride(0), _ptr(_sink128(attn_sink)), _stream(q))
    check(rc, "masked_mla_bf16")


def dsv4_masked_mla_bf16_out(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                             pref: torch.Tensor, win_lo: torch.Tensor, win_hi: torch.Tensor,
                             counts: torch.Tensor, sm_scale: float, h_per_q: int,
                             out: torch.Tensor, lse: torch.Tensor,
                             attn_sink: Optional[torch.Tensor], *, in_place_heads: bool = False,
                             detect_runs: bool = True) -> None:
    """The reference's DSv4 operator, same argument order
    (kernels/b200/dsa/litedsa_dsv4.cu:50-55): q [ng,128,d] bf16, kv [s_kv,(1,)d] bf16 flat
    workspace, indices [ng,(1,)topk] i32 ascending union rows (-1 padded, topk % 64 == 0),
    pref / win_lo / win_hi [ng,G] i32 rank ranges per token, counts [ng] i32, out
    [ng,128,512] bf16, lse [ng,128] f32, attn_sink [128] f32 or None.  d = 512 (the
    reference's width) or 576.

    ``in_place_heads``: q is the model's own ``[T, H_padded, d]`` tensor and out its
    ``[T, H_padded, 512]`` tensor with ``h_per_q`` real heads per token (unit inner stride);
    the kernel reads and writes them in place, so the pack copy of q and the unpack copy of out
    that the reference's packed path makes (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:12-22) go
    away.  lse stays packed ``[ng,128]``.

    ``detect_runs`` (default): the index lists are classified on the device and, when every
    tile's list is two contiguous runs of rows (the packed prefix + window pattern), the
    attention runs in the kernel that reads K / V with tiled TMA loads instead of gathering
    rows; otherwise in the gather kernel.  No host synchronisation either way; a small cached
    device workspace (16 + 16 * ng bytes per device) carries the decision."""
    G = 128 // int(h_per_q)
    strides = (0, 0, 0, 0)
    if in_place_heads:
        _need(q, "q", torch.bfloat16, 3)
        _need(out, "out", torch.bfloat16, 3)
        if indices.dim() == 3:
            indices = indices[:, 0]
        ng = indices.shape[0]
        d = q.shape[2]
        if q.shape[0] != ng * G or q.shape[1] < h_per_q or d not in (512, 576) or q.stride(2) != 1:
            raise ValueError("in_place_heads: q must be [ng*G, H_padded >= h_per_q, d] with unit inner stride")
        if out.shape[0] != ng * G or out.shape[1] < h_per_q or out.shape[2] != 512 or out.stride(2) != 1:
            raise ValueError("in_place_heads: out must be [ng*G, H_padded >= h_per_q, 512] with unit inner stride")
        strides = (q.stride(0), q.stride(1), out.stride(0), out.stride(1))
        q_row_stride = q.stride(1)
        _need(kv, "kv", torch.bfloat16)
        _need(indices, "indices", torch.int32)
        _need(lse, "lse", torch.float32)
        if kv.dim() == 3:
            kv = kv[:, 0]
        if kv.shape[1] != d or kv.stride(1) != 1 or indices.stride(1) != 1:
            raise ValueError("kv must be [s_kv,(1,)d] and indices [ng,(1,)topk] with unit inner stride")
        if lse.numel() != ng * 128 or not lse.is_contiguous():
            raise ValueError("lse must be a contiguous [ng,128]")
    else:
        kv, indices, ng, d = _bf16_common(q, kv, indices, out, lse)
        q_row_stride = q.stride(1)
    topk = indices.shape[1]
    for name, t in (("pref", pref), ("win_lo", win_lo), ("win_hi", win_hi)):
        _need(t, name, torch.int32)
        if t.numel() != ng * G or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous [ng, G]")
    _need(counts, "counts", torch.int32, 1)
    if counts.shape[0] != ng or not counts.is_contiguous():
        raise ValueError("counts must be a contiguous [ng]")
    ws = _runs_workspace(q.device, ng) if detect_runs else None
    with torch.cuda.device(q.device):
        rc = _lib.lib().litedsa_dsv4_masked_mla_bf16(
            _ptr(q), _ptr(kv), _ptr(indices), _ptr(pref), _ptr(win_lo), _ptr(win_hi), _ptr(counts),
            float(sm_scale), int(h_per_q), _ptr(out), _ptr(lse), _ptr(_sink128(attn_sink)), ng,
            kv.shape[0], topk, d, q_row_stride, kv.stride(0), indices.stride(0), strides[0], strides[1],
            strides[2], strides[3], _ptr(ws), 0 if ws is None else ws.numel(), _stream(q))
    check(rc, "dsv4_masked_mla_bf16")


_RUNS_WS = {}


def _runs_workspace(device: torch.device, ng: int) -> torch.Tensor:
    """Per (device, stream) byte buffer for the run classification of the DSv4 operator
    (grown on demand, reused by later calls on the same stream)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    need = 16 + 16 * int(ng)
    ws = _RUNS_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty((max(need, 1 << 16),), dtype=torch.uint8, device=device)
        _RUNS_WS[key] = ws
    return ws


def _status(fn_name: str, reset: bool, device) -> Tuple[int, int, int, int]:
    import ctypes
    buf = (ctypes.c_int * 4)()
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        torch.cuda.synchronize()
        getattr(_lib.lib(), fn_name)(buf, 1 if reset else 0)
    return tuple(int(x) for x in buf)


def attn_status(reset: bool = False, device=None) -> Tuple[int, int, int, int]:
    """Synchronise and read the FP8 attention kernels' device status block: (first wait site
    that expired since the last reset or 0, block, iteration, launches completed).  The record
    is sticky until ``reset``; an expired wait invalidates only the launch it happened in."""
    return _status("litedsa_attn_status", reset, device)


def bf16_status(reset: bool = False, device=None) -> Tuple[int, int, int, int]:
    """Status block of the bf16 gather kernel (see :func:`attn_status`)."""
    return _status("litedsa_bf16_status", reset, device)


def probe_mma_tflops(kind: str = "fp8", m_pair: int = 256, iters: int = 16384, device=None) -> float:
    """Dense tcgen05 MMA rate of the device in TFLOP/s (``kind`` "fp8" or "bf16"; ``m_pair``
    256 = peak shape, 128 = the attention kernels' 64-rows-per-CTA shape).  Synchronous."""
    import ctypes
    val = ctypes.c_double(0.0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        check(_lib.lib().litedsa_probe_mma_tflops({"fp8": 0, "bf16": 1}[kind], int(m_pair), int(iters),
                                                  ctypes.byref(val)), "probe_mma_tflops")
    return float(val.value)


def set_wait_limit_ns(limit_ns: int) -> int:
    """Limit of one device-side wait for later launches (0 = default 2 s); returns the old value."""
    import ctypes
    old = ctypes.c_uint64(0)
    check(_lib.lib().litedsa_set_wait_limit_ns(int(limit_ns), ctypes.byref(old)), "set_wait_limit_ns")
    return int(old.value)


# --------------------------------------------------------------------------- indexer + top-k
def index_logits_fp8(q_idx8: torch.Tensor, k_idx8: torch.Tensor, weights: torch.Tensor,
                     k_scale: Optional[torch.Tensor], q_pos0: int,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index logits ``[T, S]`` fp32 of the FP8 lightning indexer:
    ``k_scale[s] * sum_h weights[t,h] * relu(q_idx8[t,h,:] . k_idx8[s,:])`` for ``s <= q_pos0 + t``.

    ``q_idx8`` [T, Hi, 128] and ``k_idx8`` [S, 128] hold e4m3 codes (uint8 or float8_e4m3fn),
    ``weights`` [T, Hi] fp32, ``k_scale`` [S] fp32 or None.  Entries beyond a token's position
    are written as -inf (``topk_select`` never reads them).
    """
    for t, n in ((q_idx8, "q_idx8"), (k_idx8, "k_idx8")):
        if not t.is_cuda or t.element_size() != 1:
            raise TypeError(f"{n} must be a CUDA tensor of 1-byte e4m3 codes")
    _need(weights, "weights", torch.float32, 2)
    if q_idx8.dim() != 3 or q_idx8.shape[2] != 128 or not q_idx8.is_contiguous():
        raise ValueError("q_idx8 must be a contiguous [T, Hi, 128] tensor")
    if k_idx8.dim() != 2 or k_idx8.shape[1] != 128 or k_idx8.stride(1) != 1:
        raise ValueError("k_idx8 must be [S, 128] with unit inner stride")
    T, Hi, _ = q_idx8.shape
    S = k_idx8.shape[0]
    if tuple(weights.shape) != (T, Hi) or not weights.is_contiguous():
        raise ValueError("weights must be a contiguous [T, Hi] tensor")
    if k_scale is not None:
        _need(k_scale, "k_scale", torch.float32, 1)
        if k_scale.numel() != S or not k_scale.is_contiguous():
            raise ValueError("k_scale must be a contiguous [S] tensor")
    if out is None:
        out = torch.empty((T, S), dtype=torch.float32, device=q_idx8.device)
    _need(out, "out", torch.float32, 2)
    if out.shape[0] != T or out.shape[1] < S or out.stride(1) != 1:
        raise ValueError("out must be [T, >= S] fp32 with unit inner stride")
    with torch.cuda.device(q_idx8.device):
        check(_lib.lib().litedsa_index_logits_fp8(_ptr(q_idx8), _ptr(k_idx8), _ptr(weights), _ptr(k_scale),
                                                  _ptr(out), T, Hi, S, int(q_pos0), k_idx8.stride(0),
                                                  out.stride(0), _stream(q_idx8)), "index_logits_fp8")
    return out


def topk_select(logits: torch.Tensor, k: int, *, q_pos0: int = 0, lengths: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact top-``k`` positions of every row of ``logits`` [T, S] fp32 among its first
    ``lengths[t]`` entries (default: causal, ``min(S, q_pos0 + t + 1)``): the selected set is
    exact (ties at the k-th value towards smaller positions), the order inside a row is not
    specified, short rows are padded with -1 at the end.  The result is the ``topk_idx`` tensor
    ``union_qm`` takes."""
    _need(logits, "logits", torch.float32, 2)
    if logits.stride(1) != 1:
        raise ValueError("logits must have unit inner stride")
    T, S = logits.shape
    if lengths is not None:
        _need(lengths, "lengths", torch.int32, 1)
        if lengths.numel() != T or not lengths.is_contiguous():
            raise ValueError("lengths must be a contiguous [T] int32 tensor")
    if out is None:
        out = torch.empty((T, int(k)), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 2)
    if tuple(out.shape) != (T, int(k)) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [T, k] int32 tensor")
    with torch.cuda.device(logits.device):
        check(_lib.lib().litedsa_topk_select(_ptr(logits), _ptr(lengths), _ptr(out), T, S, int(k),
                                             int(q_pos0), logits.stride(0), _stream(logits)), "topk_select")
    return out


def lite_topk(q_idx8: torch.Tensor, k_idx8: torch.Tensor, weights: torch.Tensor,
              k_scale: Optional[torch.Tensor], k: int, q_pos0: int, *,
              logits_workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indexer + selection in one call: ``topk_idx`` [T, k] int32 (-1 padded) for the T query
    tokens at positions ``q_pos0 ...`` -- the input of ``union_qm`` / ``sparse_prefill``."""
    logits = index_logits_fp8(q_idx8, k_idx8, weights, k_scale, q_pos0, out=logits_workspace)
    S = k_idx8.shape[0]
    # a workspace wider than S: select over the first S columns of every row
    view = logits if logits.shape[1] == S else logits.as_strided((logits.shape[0], S), (logits.stride(0), 1))
    return topk_select(view, k, q_pos0=q_pos0)


def index_status(reset: bool = False, device=None) -> Tuple[int, int, int, int]:
    """Status word of the index-logits kernel (see :func:`attn_status`)."""
    return _status("litedsa_index_status", reset, device)


# --------------------------------------------------------------------------- operand preparation
def quantize_e4m3(x: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """e4m3 codes (uint8) of ``x / scale`` for a contiguous bf16 CUDA tensor (saturating)."""
    _need(x, "x", torch.bfloat16)
    if not x.is_contiguous() or x.numel() % 8:
        raise ValueError("x must be contiguous with a multiple of 8 elements")
    if out is None:
        out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    else:
        _need(out, "out", (torch.uint8, torch.float8_e4m3fn))
        if out.numel() != x.numel() or not out.is_contiguous():
            raise ValueError("out must be contiguous and match x")
    with torch.cuda.device(x.device):
        check(_lib.lib().litedsa_quantize_e4m3(_ptr(x), _ptr(out), x.numel(), float(scale),
                                               _stream(x)), "quantize_e4m3")
    return out


def repack_kv656(kv_rows: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None,
                 *, check_scales: bool = False, return_flag: bool = False):
    """Packed 656-byte cache rows -> ``[s_kv, 576]`` e4m3 codes sharing the scalar ``scale``.

    Only caches whose per-128 scales all equal ``scale`` have this form.  The kernel sets a
    device flag when some scale differs: ``return_flag`` returns ``(out, flag)`` (flag: int32
    [1] on the device, non-zero = mismatch; no host synchronisation), ``check_scales`` reads
    it back (one device->host read) and raises.  Caches with differing scales go through
    :func:`dequant_kv656` and the bf16 kernel instead."""
    _need(kv_rows, "kv_rows", torch.uint8, 2)
    if kv_rows.shape[1] != 656 or not kv_rows.is_contiguous():
        raise ValueError("kv_rows must be a contiguous [s_kv, 656] uint8 tensor")
    s_kv = kv_rows.shape[0]
    if out is None:
        out = torch.empty((s_kv, 576), dtype=torch.uint8, device=kv_rows.device)
    flag = torch.zeros((1,), dtype=torch.int32, device=kv_rows.device)
    with torch.cuda.device(kv_rows.device):
        check(_lib.lib().litedsa_repack_kv656(_ptr(kv_rows), _ptr(out), s_kv, out.stride(0),
                                              float(scale), _ptr(flag), _stream(kv_rows)),
              "repack_kv656")
    if check_scales and int(flag.item()) != 0:
        raise ValueError("the cache has per-128 scales different from `scale`; it cannot be "
                         "expressed with one scalar scale (use dequant_kv656 + the bf16 path)")
    return (out, flag) if return_flag else out


def dequant_kv656(kv_rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed 656-byte cache rows -> bf16 ``[s_kv, 576]`` (codes x per-128 scales ‖ rope): the
    flat workspace the bf16 kernel gathers from."""
    _need(kv_rows, "kv_rows", torch.uint8, 2)
    if kv_rows.shape[1] != 656 or not kv_rows.is_contiguous():
        raise ValueError("kv_rows must be a contiguous [s_kv, 656] uint8 tensor")
    s_kv = kv_rows.shape[0]
    if out is None:
        out = torch.empty((s_kv, 576), dtype=torch.bfloat16, device=kv_rows.device)
    else:
        _need(out, "out", torch.bfloat16, 2)
        if tuple(out.shape) != (s_kv, 576) or out.stride(1) != 1:
            raise ValueError("out must be [s_kv, 576] bf16 with unit inner stride")
    with torch.cuda.device(kv_rows.device):
        check(_lib.lib().litedsa_dequant_kv656(_ptr(kv_rows), _ptr(out), s_kv, out.stride(0) * 2,
                                               _stream(kv_rows)), "dequant_kv656")
    return out


def merge_kv_splits(out_parts: torch.Tensor, lse_parts: torch.Tensor, q_group_div: int, *,
                    max_parts: Optional[torch.Tensor] = None,
                    attn_sink: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    lse: Optional[torch.Tensor] = None):
    """Combine the outputs of ``q_group_div`` consecutive tiles that shared one Q tile
    (:func:`masked_mla_fp8_out` with ``q_group_div > 1``: slices of one long union list) into
    the attention over the whole list.

    ``out_parts`` [ng,128,512] bf16, ``lse_parts`` [ng,128] f32 (+inf marks a slice without
    keys), ``max_parts`` [ng,128] optional, ``attn_sink`` [128] f32: the array the attention
    call got.  Returns ``(out [ng/div,128,512] bf16, lse [ng/div,128] f32)`` and, with
    ``max_parts``, the merged ``max_logits``.  The reference leaves this step to its callers
    (kernels/b200/dsa/litedsa_attention_sm100.cuh:1383-1385).
    """
    _need(out_parts, "out_parts", torch.bfloat16, 3)
    _need(lse_parts, "lse_parts", torch.float32, 2)
    ng = out_parts.shape[0]
    div = int(q_group_div)
    if tuple(out_parts.shape) != (ng, 128, 512) or tuple(lse_parts.shape) != (ng, 128) \
            or not out_parts.is_contiguous() or not lse_parts.is_contiguous():
        raise ValueError("out_parts must be contiguous [ng,128,512] bf16 and lse_parts [ng,128] f32")
    if div < 1 or ng % div:
        raise ValueError("q_group_div must divide the number of tiles")
    dev = out_parts.device
    for name, t in (("max_parts", max_parts), ("attn_sink", attn_sink)):
        if t is not None:
            _need(t, name, torch.float32, 2 if name == "max_parts" else 1)
            if t.device != dev or not t.is_contiguous() or \
                    tuple(t.shape) != ((ng, 128) if name == "max_parts" else (128,)):
                raise ValueError(f"{name} has the wrong shape, layout or device")
    nm = ng // div
    if out is None:
        out = torch.empty((nm, 128, 512), dtype=torch.bfloat16, device=dev)
    if lse is None:
        lse = torch.empty((nm, 128), dtype=torch.float32, device=dev)
    if tuple(out.shape) != (nm, 128, 512) or out.dtype != torch.bfloat16 or not out.is_contiguous() \
            or tuple(lse.shape) != (nm, 128) or lse.dtype != torch.float32 or not lse.is_contiguous() \
            or out.device != dev or lse.device != dev:
        raise ValueError("out must be contiguous [ng/div,128,512] bf16 and lse [ng/div,128] f32")
    mx = torch.empty((nm, 128), dtype=torch.float32, device=dev) if max_parts is not None else None
    with torch.cuda.device(dev):
        check(_lib.lib().litedsa_merge_kv_splits(_ptr(out_parts), _ptr(lse_parts), _ptr(max_parts),
                                                 _ptr(attn_sink), _ptr(out), _ptr(lse), _ptr(mx),
                                                 ng, div, _stream(out_parts)), "merge_kv_splits")
    return (out, lse, mx) if max_parts is not None else (out, lse)


def prepare_kv(kv_cache_fp8: torch.Tensor, kv_scale: Optional[float] = None,
               *, check_scales: bool = False) -> torch.Tensor:
    """Bring a KV cache into the form one of the attention kernels gathers from.

    * ``[s_kv, 576]`` e4m3 / uint8 codes (one scalar scale) or a bf16 ``[s_kv, 576]``
      workspace: returned as is.
    * packed ``[s_kv, 656]`` uint8 rows with ``kv_scale`` given: the caller states that every
      per-128 scale equals ``kv_scale`` -> repacked to ``[s_kv, 576]`` codes (FP8 kernel).
    * packed rows with ``kv_scale`` None: per-128 scales may differ (a DeepSeek-V3.2 cache)
      -> dequantised to a bf16 ``[s_kv, 576]`` workspace (bf16 kernel).
    Do this once per cache and hand the result to :func:`masked_mla_fp8` / :func:`sparse_prefill`.
    """
    kv = kv_cache_fp8
    if kv.dim() == 2 and kv.shape[1] == 656 and kv.dtype == torch.uint8:
        return dequant_kv656(kv) if kv_scale is None else repack_kv656(kv, kv_scale, check_scales=check_scales)
    return kv


def masked_mla_fp8(q: torch.Tensor, kv_cache_fp8: torch.Tensor, union_idx: torch.Tensor,
                   mask: torch.Tensor, sm_scale: float, *, counts: Optional[torch.Tensor] = None,
                   kv_scale: Optional[float] = None, q_scale: Optional[float] = None,
                   return_max_logits: bool = False, out: Optional[torch.Tensor] = None,
                   lse: Optional[torch.Tensor] = None):
    """Masked MLA prefill over the per-tile union of an FP8 KV cache; returns
    ``(out [T,h,512] bf16, lse [T,h] f32)`` (written into ``out`` / ``lse`` when given:
    contiguous, same shapes and dtypes).

    q            [T, h, 576] bf16, or e4m3/uint8 codes (FP8 route only).  G = 128 // h adjacent
                 tokens form one tile.
    kv_cache_fp8 any form :func:`prepare_kv` accepts.  Packed 656-byte rows with ``kv_scale``
                 None, or a bf16 workspace, take the **bf16 route** (per-128 scales may differ;
                 bf16 tensor-core MMAs, bf16 P: accurate to bf16 rounding).  e4m3 codes, or
                 packed rows with a stated uniform ``kv_scale``, take the **FP8 route** (the
                 reference kernel's numerics: q, K, V and P in e4m3, fp32 accumulation).
    union_idx    [T/G, G*k] int32 and mask [T/G, G, G*k/32] from :func:`union_qm`;
                 counts [T/G] int32 (default: entries before the -1 padding, one extra pass).
    q_scale      FP8 route with bf16 q: the power-of-two quantisation scale.  When omitted it
                 is derived from max|q| with ONE host synchronisation; pass it on a hot path.
    """
    _need(q, "q", (torch.bfloat16, torch.uint8, torch.float8_e4m3fn), 3)
    T, h, d = q.shape
    if d != 576 or 128 % h or 128 // h > 16:
        raise ValueError("q must be [T, h, 576] with h dividing 128 and 128/h <= 16")
    G = 128 // h
    if T % G:
        raise ValueError("token count must be a multiple of 128 // heads")
    ng = T // G
    kv = prepare_kv(kv_cache_fp8, kv_scale)
    if counts is None:
        counts = (union_idx >= 0).sum(dim=1, dtype=torch.int32)
    if out is None:
        out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=q.device)
    else:
        _need(out, "out", torch.bfloat16)
        if out.numel() != T * h * 512 or not out.is_contiguous():
            raise ValueError("out must be a contiguous [T,h,512] bf16 tensor")
        out = out.view(ng, 128, 512)
    if lse is None:
        lse = torch.empty((ng, 128), dtype=torch.float32, device=q.device)
    else:
        _need(lse, "lse", torch.float32)
        if lse.numel() != T * h or not lse.is_contiguous():
            raise ValueError("lse must be a contiguous [T,h] f32 tensor")
        lse = lse.view(ng, 128)
    ml = torch.empty((ng, 128), dtype=torch.float32, device=q.device) if return_max_logits else None
    if kv.dtype == torch.bfloat16:
        if q.dtype != torch.bfloat16:
            raise TypeError("the bf16 route (cache with per-128 scales / bf16 workspace) needs bf16 q")
        masked_mla_bf16_out(q.contiguous().view(ng, 128, 576), kv, union_idx, float(sm_scale), counts,
                            mask, h, out, ml, lse)
    else:
        ks = 1.0 if kv_scale is None else float(kv_scale)
        if q.dtype == torch.bfloat16:
            if q_scale is None:      # convenience: one device->host read
                amax = float(q.abs().amax().item())
                q_scale = 2.0 ** max(-24, int(torch.tensor(max(amax, 1e-30) / 448.0).log2().ceil().item()))
            q8 = quantize_e4m3(q.contiguous(), q_scale)
        else:
            q8 = q.contiguous()
            q_scale = 1.0 if q_scale is None else q_scale
        masked_mla_fp8_out(q8.view(ng, 128, 576), kv, union_idx, float(sm_scale) * q_scale * ks,
                           ks, counts, mask, h, out, ml, lse)
    res = (out.view(T, h, 512), lse.view(T, h))
    return res + (ml.view(T, h),) if return_max_logits else res


def sparse_prefill(q: torch.Tensor, kv_cache_fp8: torch.Tensor, topk_idx: torch.Tensor,
                   sm_scale: float, *, kv_scale: Optional[float] = None,
                   q_scale: Optional[float] = None, seq_space: Optional[int] = None,
                   out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None):
    """The whole hot path for one chunk of query tokens: union_qm + masked attention.

    q [T,h,576], topk_idx [T,k] int32, kv_cache_fp8 as in :func:`masked_mla_fp8` (already
    resident on the device; pass the result of :func:`prepare_kv` when the same cache serves
    several calls).  Returns ``(out [T,h,512] bf16, lse [T,h] f32)``, written into ``out`` /
    ``lse`` when given.
    """
    h = q.shape[1]
    u, m, c = union_qm(topk_idx, 128 // h,
                       seq_space=seq_space if seq_space is not None else kv_cache_fp8.shape[0],
                       return_counts=True)
    return masked_mla_fp8(q, kv_cache_fp8, u, m, sm_scale, counts=c, kv_scale=kv_scale,
                          q_scale=q_scale, out=out, lse=lse)


_SIDE_STREAMS = {}
_HOST_WORKSPACE = {}


def _side_streams(device: torch.device):
    """One (upload, download) stream pair per device, created on first use."""
    key = torch.device(device).index if torch.device(device).index is not None \
        else torch.cuda.current_device()
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = (torch.cuda.Stream(device=key), torch.cuda.Stream(device=key))
    return _SIDE_STREAMS[key]


def _host_workspace(device, T: int, h: int, k: int, q_dtype, idx_dtype):
    """Device staging buffers of :func:`sparse_prefill_host`, kept per (device, shape) so that
    steady-state calls allocate nothing (one q + top-k + out + lse image of the step)."""
    key = (str(device), T, h, k, q_dtype, idx_dtype)
    ws = _HOST_WORKSPACE.get(key)
    if ws is None:
        _HOST_WORKSPACE.clear()            # one live shape per process is enough
        ws = (torch.empty((T, h, 576), dtype=q_dtype, device=device),
              torch.empty((T, k), dtype=idx_dtype, device=device),
              torch.empty((T, h, 512), dtype=torch.bfloat16, device=device),
              torch.empty((T, h), dtype=torch.float32, device=device))
        _HOST_WORKSPACE[key] = ws
    return ws


def _chunk_schedule(T: int, chunk: int, G: int):
    """Token bounds of the pipelined chunks: full chunks in the middle, a quarter and a half
    chunk at either end.  The first upload and the last download are the two copies nothing
    overlaps, so they are kept short."""
    ramp = [max(G, chunk // 4 // G * G), max(G, chunk // 2 // G * G)]
    if T < 4 * chunk:
        ramp = []
    head = sum(ramp)
    bounds = [0]
    for r in ramp:
        bounds.append(bounds[-1] + r)
    tail_start = T - head
    while bounds[-1] + chunk <= tail_start:
        bounds.append(bounds[-1] + chunk)
    if bounds[-1] < tail_start:
        bounds.append(tail_start)
    for r in reversed(ramp):
        bounds.append(bounds[-1] + r)
    if not ramp and bounds[-1] != T:
        bounds.append(T)
    return bounds


def sparse_prefill_host(q_host: torch.Tensor, kv_cache_fp8: torch.Tensor, topk_host: torch.Tensor,
                        sm_scale: float, *, out_host: Optional[torch.Tensor] = None,
                        lse_host: Optional[torch.Tensor] = None, kv_scale: Optional[float] = None,
                        q_scale: Optional[float] = None, seq_space: Optional[int] = None,
                        chunk_tokens: int = 512):
    """:func:`sparse_prefill` for callers whose queries and results live in host memory.

    ``q_host`` [T,h,576] and ``topk_host`` [T,k] are host tensors (pinned for full speed),
    ``kv_cache_fp8`` is resident on the device.  The tokens are cut into tile-aligned chunks
    and pipelined over three streams: the upload of chunk i+1, the kernels of chunk i (on
    the caller's current stream) and the download of chunk i-1 run concurrently, so a step
    costs about max(upload, download) instead of their sum plus the kernels (the first and
    the last chunks are shorter: their upload / download is not overlapped).  Results are
    written to ``out_host`` [T,h,512] bf16 and ``lse_host`` [T,h] f32 (allocated pinned when
    not given); they are complete once the caller's current stream has been synchronised.
    The device staging buffers are cached per shape (see :func:`_host_workspace`); calls on
    one device must not overlap each other.
    """
    if q_host.is_cuda or topk_host.is_cuda:
        raise ValueError("q_host and topk_host must be host tensors (use sparse_prefill)")
    if not kv_cache_fp8.is_cuda:
        raise ValueError("kv_cache_fp8 must be resident on a CUDA device (there is no CPU path)")
    if q_host.dim() != 3 or q_host.shape[2] != 576 or topk_host.dim() != 2 \
            or topk_host.shape[0] != q_host.shape[0]:
        raise ValueError("q_host must be [T,h,576] and topk_host [T,k]")
    T, h, _ = q_host.shape
    if 128 % h or 128 // h > 16 or T % (128 // h):
        raise ValueError("heads must divide 128 (128/h <= 16) and T be a multiple of 128 // heads")
    G = 128 // h
    dev = kv_cache_fp8.device
    chunk = max(G, int(chunk_tokens) // G * G)
    if out_host is None:
        out_host = torch.empty((T, h, 512), dtype=torch.bfloat16).pin_memory()
    if lse_host is None:
        lse_host = torch.empty((T, h), dtype=torch.float32).pin_memory()
    if tuple(out_host.shape) != (T, h, 512) or out_host.dtype != torch.bfloat16 or \
            tuple(lse_host.shape) != (T, h) or lse_host.dtype != torch.float32:
        raise ValueError("out_host must be [T,h,512] bf16 and lse_host [T,h] f32")
    space = seq_space if seq_space is not None else kv_cache_fp8.shape[0]
    with torch.cuda.device(dev):
        kv = prepare_kv(kv_cache_fp8, kv_scale)       # once per call, not per chunk
        if kv.dtype != torch.bfloat16 and q_host.dtype == torch.bfloat16 and q_scale is None:
            raise ValueError("bf16 queries on the FP8 route need q_scale (no host synchronisation "
                             "happens inside the pipelined chunks)")
        qd, idd, od, ld = _host_workspace(dev, T, h, topk_host.shape[1], q_host.dtype,
                                          topk_host.dtype)
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = _side_streams(dev)
        s_in.wait_stream(cur)      # earlier kernels may still read the staging buffers
        s_out.wait_stream(cur)
        bounds = _chunk_schedule(T, chunk, G)
        for t0, t1 in zip(bounds[:-1], bounds[1:]):
            with torch.cuda.stream(s_in):
                qd[t0:t1].copy_(q_host[t0:t1], non_blocking=True)
                idd[t0:t1].copy_(topk_host[t0:t1], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            cur.wait_event(ev_in)
            sparse_prefill(qd[t0:t1], kv, idd[t0:t1], sm_scale, kv_scale=kv_scale, q_scale=q_scale,
                           seq_space=space, out=od[t0:t1], lse=ld[t0:t1])
            ev_c = torch.cuda.Event()
            ev_c.record(cur)
            s_out.wait_event(ev_c)
            with torch.cuda.stream(s_out):
                out_host[t0:t1].copy_(od[t0:t1], non_blocking=True)
                lse_host[t0:t1].copy_(ld[t0:t1], non_blocking=True)
        cur.wait_stream(s_out)
    return out_host, lse_host


# --------------------------------------------------------------------------- DSv4 BF16 two-range attention
def dsv4_c128a_bf16(q: torch.Tensor, kv_compressed: Optional[torch.Tensor], kv_raw: torch.Tensor,
                    q_pos0: int, sm_scale: float, *, window: int = 128, ratio: int = 128,
                    attn_sink: Optional[torch.Tensor] = None, heads: Optional[int] = None,
                    out: Optional[torch.Tensor] = None):
    """Packed BF16 attention over (compressed prefix, sliding window).

    q [T,h,576] bf16 for T consecutive tokens starting at position ``q_pos0``; token at
    position p attends to kv_compressed rows [0, p // ratio) and kv_raw rows
    [p - window + 1, p]; V = first 512 dims of the same rows.  ``attn_sink`` [h] fp32 adds
    exp(sink) to the output normaliser.  Returns ``(out [T,h,512] bf16, lse [T,h] f32)``.
    The reference's counterpart takes a gathered index list plus rank ranges
    (kernels/b200/dsa/litedsa_dsv4.cu:50-55); here the ranges are contiguous memory.

    ``heads`` (zero-copy for tensor-parallel callers): q is ``[T, H_padded, 576]`` of which only
    the first ``heads`` head slots per token are real; it is read in place (any strides with unit
    inner stride), and the result is written in place into ``out`` ``[T, H_padded, 512]`` when
    given (else a dense ``[T, heads, 512]`` is returned).  lse is ``[T, heads]``.
    """
    _need(q, "q", torch.bfloat16, 3)
    _need(kv_raw, "kv_raw", torch.bfloat16, 2)
    T, hq, d = q.shape
    h = hq if heads is None else int(heads)
    if d != 576 or h > hq or 128 % h or 128 // h > 16 or kv_raw.shape[1] != 576:
        raise ValueError("q must be [T,h,576] (h | 128, 128/h <= 16) and kv_raw [S,576]")
    G = 128 // h
    if T % G:
        raise ValueError("token count must be a multiple of 128 // heads")
    if heads is None:
        q = q.contiguous()
    elif q.stride(2) != 1:
        raise ValueError("q needs unit inner stride")
    n_comp = 0
    if kv_compressed is not None and kv_compressed.shape[0] > 0:
        _need(kv_compressed, "kv_compressed", torch.bfloat16, 2)
        if kv_compressed.shape[1] != 576 or kv_compressed.stride(1) != 1:
            raise ValueError("kv_compressed must be [Nc,576] with unit inner stride")
        n_comp = kv_compressed.shape[0]
    if kv_raw.stride(1) != 1:
        raise ValueError("kv_raw needs unit inner stride")
    sink = None
    if attn_sink is not None:
        _need(attn_sink, "attn_sink", torch.float32, 1)
        if attn_sink.shape[0] != h:
            raise ValueError("attn_sink must be [heads]")
        sink = attn_sink.repeat(G).contiguous()            # per packed row
    ng = T // G
    in_place_out = out is not None
    if in_place_out:
        _need(out, "out", torch.bfloat16, 3)
        if out.shape[0] != T or out.shape[1] < h or out.shape[2] != 512 or out.stride(2) != 1:
            raise ValueError("out must be [T, H_padded >= heads, 512] with unit inner stride")
    else:
        out = torch.empty((T, h, 512), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        rc = _lib.lib().litedsa_dsv4_c128a_bf16(
            _ptr(q), _ptr(kv_compressed) if n_comp else None, _ptr(kv_raw), ng, h, n_comp,
            kv_raw.shape[0], int(q_pos0), int(window), int(ratio), float(sm_scale), _ptr(sink),
            _ptr(out), _ptr(lse), q.stride(1), kv_compressed.stride(0) if n_comp else 576, kv_raw.stride(0),
            q.stride(0), q.stride(1), out.stride(0), out.stride(1), _stream(q))
    check(rc, "dsv4_c128a_bf16")
    return out, lse.view(T, h)


def dsv4_status(reset: bool = False, device=None) -> Tuple[int, int, int, int]:
    """Status word of the DSv4 kernel (see :func:`attn_status`)."""
    import ctypes
    buf = (ctypes.c_int * 4)()
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        torch.cuda.synchronize()
        _lib.lib().litedsa_dsv4_status(buf, 1 if reset else 0)
    return tuple(int(x) for x in buf)
