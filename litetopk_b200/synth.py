"""Seeded synthetic workloads for the LiteDSA sparse-attention hot path.

The reference ships no dataset, benchmark script or fixture for this path, so the
five workload shapes below (taken from the benchmark definition this package is
measured on) are generated here from a seed.  They stand in for real top-k
selections and KV caches; only shapes, sizes and value distributions matter.

Top-k lists: the G adjacent tokens that share one 128-row tile draw a fraction
``f`` of their k indices from a pool shared by the tile and the rest privately, so
the size of the per-tile union is ``round(f*k) + G*(k - round(f*k))``.  All
indices are causal (<= the first position of the tile), each token's list is
randomly permuted, and lists that cannot be filled are padded with -1.

KV cache, "native" mode (DeepSeek-V3.2 cache row, 656 bytes):
    bytes [0, 512)    e4m3 codes of the 512-dim latent,
    bytes [512, 528)  four fp32 scales, one per 128 latent dims (amax / 448),
    bytes [528, 656)  the 64-dim rope part as bf16.
"ref-compatible" mode draws the same tensors but forces every per-128 scale to one
power of two and rounds q and the rope part to the e4m3 grid, so that the very same
operands can also be handed to a kernel that takes a 576-wide all-e4m3 cache with a
single scalar scale (the layout the reference module consumes,
kernels/b200/dsa/litedsa.cu:82-92).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Tuple

import torch

E4M3_MAX = 448.0
KV_ROW_BYTES = 656
D_LATENT = 512
D_ROPE = 64
D_QK = D_LATENT + D_ROPE
REFCOMPAT_SCALE = 2.0 ** -6  # one shared power-of-two scale for q, latent and rope


@dataclasses.dataclass(frozen=True)
class Workload:
    """Shape of one benchmark configuration."""

    name: str
    tokens: int            # query tokens T
    heads: int             # q heads per token (G = 128 // heads tokens share a tile)
    topk: int              # k indices per token (0 for the DSv4 range workload)
    s_kv: int              # KV cache length; queries sit at its tail
    overlap: Tuple[float, float]  # per-tile shared fraction f drawn uniformly in [lo, hi]
    kind: str = "fp8"      # "fp8" (union + masked FP8 MLA) or "dsv4" (bf16 two-range)
    n_compressed: int = 0  # dsv4 only: entries in the compressed KV
    window: int = 128      # dsv4 only
    ratio: int = 128       # dsv4 only

    @property
    def group(self) -> int:
        return 128 // self.heads

    @property
    def tiles(self) -> int:
        return self.tokens // self.group

    @property
    def cap(self) -> int:
        return self.group * self.topk

    @property
    def pos0(self) -> int:
        return self.s_kv - self.tokens


CONFIGS = {
    # config 0: the CPU-sized correctness case
    "c0": Workload("c0", tokens=256, heads=64, topk=512, s_kv=4096, overlap=(0.80, 0.80)),
    # config 1: the headline single-GPU FP8 prefill case
    "c1": Workload("c1", tokens=8192, heads=64, topk=2048, s_kv=32768, overlap=(0.75, 0.75)),
    # config 2: 32 heads (4 tokens per tile), variable union size
    "c2": Workload("c2", tokens=16384, heads=32, topk=1024, s_kv=65536, overlap=(0.50, 0.90)),
    # config 3: DeepSeek-V4 style packed BF16 compressed-prefix + sliding-window attention
    "c3": Workload("c3", tokens=16384, heads=64, topk=0, s_kv=131072, overlap=(0.0, 0.0),
                   kind="dsv4", n_compressed=1024),
    # config 4: the multi-GPU long-context case (16 heads, 8 tokens per tile)
    "c4": Workload("c4", tokens=65536, heads=16, topk=2048, s_kv=131072, overlap=(0.70, 0.70)),
}


def scaled(w: Workload, *, tokens: Optional[int] = None, s_kv: Optional[int] = None,
           topk: Optional[int] = None) -> Workload:
    """A smaller workload with the same structure (used by tests and CPU baselines)."""
    return dataclasses.replace(
        w, tokens=tokens if tokens is not None else w.tokens,
        s_kv=s_kv if s_kv is not None else w.s_kv,
        topk=topk if topk is not None else w.topk)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


TOPK_GRANULE = 64  # tiles generated from one RNG stream


def _topk_granule(w: Workload, seed: int, granule: int, f_all: torch.Tensor, device) -> torch.Tensor:
    """Lists of the tiles [granule*64, granule*64+64) as ``[n, G, k]`` int64."""
    G, k = w.group, w.topk
    t0 = granule * TOPK_GRANULE
    t1 = min(w.tiles, t0 + TOPK_GRANULE)
    n = t1 - t0
    tile_id = torch.arange(t0, t1, device=device)
    p0 = (w.pos0 + tile_id * G).to(torch.int64)                        # first position of the tile
    f = f_all[t0:t1].to(device)
    n_pool = torch.round(f.double() * k).to(torch.int64)               # shared entries per token
    n_extra = k - n_pool
    need = min(int((n_pool + G * n_extra).max().item()), w.s_kv)
    g_dev = _gen(seed * 7919 + granule * 31 + 1, device)
    keys = torch.rand((n, w.s_kv), generator=g_dev, device=device)
    pos = torch.arange(w.s_kv, device=device)[None, :]
    keys = torch.where(pos <= p0[:, None], keys, torch.full_like(keys, 2.0))
    order = torch.topk(keys, need, dim=1, largest=False, sorted=True).indices  # random distinct causal positions
    avail = (p0 + 1).clamp(max=w.s_kv)
    slot = torch.arange(need, device=device)[None, :]
    order = torch.where(slot < avail[:, None], order, torch.full_like(order, -1))
    j = torch.arange(k, device=device)[None, None, :]                   # [1,1,k]
    q = torch.arange(G, device=device)[None, :, None]                   # [1,G,1]
    npool = n_pool[:, None, None]
    src = torch.where(j < npool, j.expand(n, G, k),
                      npool + q * n_extra[:, None, None] + (j - npool))
    valid_src = src < need
    src = src.clamp(max=need - 1)
    lists = torch.gather(order[:, None, :].expand(n, G, need), 2, src)
    lists = torch.where(valid_src, lists, torch.full_like(lists, -1))
    shuffle = torch.rand((n, G, k), generator=g_dev, device=device).argsort(dim=2)
    return torch.gather(lists, 2, shuffle)


def make_topk(w: Workload, seed: int = 0, device="cpu", first_tile: int = 0,
              num_tiles: Optional[int] = None) -> torch.Tensor:
    """Top-k index lists ``[num_tiles*G, k]`` int32 for tiles [first_tile, first_tile+num_tiles).

    Tiles are generated in granules of 64 from ``(seed, granule number)`` only, so a rank
    that owns a slice of the tiles generates exactly the rows the single-rank run would.
    """
    G, k = w.group, w.topk
    n_t = w.tiles - first_tile if num_tiles is None else num_tiles
    out = torch.empty((n_t * G, k), dtype=torch.int32, device=device)
    gen = _gen(seed * 1000003 + 17, "cpu")
    # per-tile overlap fraction, drawn for ALL tiles so slices agree with the full run
    f_all = torch.rand(w.tiles, generator=gen) * (w.overlap[1] - w.overlap[0]) + w.overlap[0]
    last = first_tile + n_t
    for gr in range(first_tile // TOPK_GRANULE, (last + TOPK_GRANULE - 1) // TOPK_GRANULE):
        lists = _topk_granule(w, seed, gr, f_all, device)
        g0 = gr * TOPK_GRANULE
        lo, hi = max(first_tile, g0), min(last, g0 + lists.shape[0])
        out[(lo - first_tile) * G:(hi - first_tile) * G] = \
            lists[lo - g0:hi - g0].reshape((hi - lo) * G, k).to(torch.int32)
    return out


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 values to the e4m3 grid (saturating at +-448), returned as fp32."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()


def e4m3_codes(x: torch.Tensor) -> torch.Tensor:
    """e4m3 byte codes (uint8) of fp32 values, saturating at +-448."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def make_kv_cache(s_kv: int, seed: int = 0, device="cpu", mode: str = "native") -> torch.Tensor:
    """Packed FP8 KV cache ``[s_kv, 656]`` uint8 (layout in the module docstring)."""
    gen = _gen(seed * 104729 + 3, device)
    latent = torch.randn((s_kv, D_LATENT), generator=gen, device=device)
    rope = torch.randn((s_kv, D_ROPE), generator=gen, device=device)
    lat4 = latent.view(s_kv, 4, 128)
    if mode == "native":
        scale = lat4.abs().amax(dim=2).clamp_min(1e-8) / E4M3_MAX          # [s_kv, 4] fp32
    elif mode == "refcompat":
        scale = torch.full((s_kv, 4), REFCOMPAT_SCALE, device=device)
        rope = e4m3_round(rope / REFCOMPAT_SCALE) * REFCOMPAT_SCALE
    else:
        raise ValueError(f"unknown KV mode {mode!r}")
    codes = e4m3_codes(lat4 / scale[:, :, None]).view(s_kv, D_LATENT)
    row = torch.empty((s_kv, KV_ROW_BYTES), dtype=torch.uint8, device=device)
    row[:, :D_LATENT] = codes
    row[:, D_LATENT:D_LATENT + 16] = scale.float().contiguous().view(torch.uint8).view(s_kv, 16)
    row[:, D_LATENT + 16:] = rope.to(torch.bfloat16).contiguous().view(torch.uint8).view(s_kv, 128)
    return row


def make_q(tokens: int, heads: int, seed: int = 0, device="cpu", mode: str = "native",
           d: int = D_QK) -> torch.Tensor:
    """Queries ``[tokens, heads, d]`` bf16 ~ N(0,1) (on the e4m3 grid in refcompat mode)."""
    gen = _gen(seed * 15485863 + 5, device)
    q = torch.randn((tokens, heads, d), generator=gen, device=device)
    if mode == "refcompat":
        q = e4m3_round(q / REFCOMPAT_SCALE) * REFCOMPAT_SCALE
    return q.to(torch.bfloat16)


def split_kv_cache(kv_rows: torch.Tensor):
    """Views of a packed cache: (codes [s,512] u8, scales [s,4] f32, rope [s,64] bf16)."""
    s = kv_rows.shape[0]
    codes = kv_rows[:, :D_LATENT]
    scales = kv_rows[:, D_LATENT:D_LATENT + 16].contiguous().view(torch.float32).view(s, 4)
    rope = kv_rows[:, D_LATENT + 16:].contiguous().view(torch.bfloat16).view(s, D_ROPE)
    return codes, scales, rope


def dequant_kv_cache(kv_rows: torch.Tensor) -> torch.Tensor:
    """fp32 ``[s_kv, 576]`` values of a packed cache (latent codes x scales ‖ rope)."""
    codes, scales, rope = split_kv_cache(kv_rows)
    s = kv_rows.shape[0]
    lat = codes.contiguous().view(torch.float8_e4m3fn).float().view(s, 4, 128) * scales[:, :, None]
    return torch.cat([lat.view(s, D_LATENT), rope.float()], dim=1)


def refcompat_operands(q: torch.Tensor, kv_rows: torch.Tensor):
    """All-e4m3 operands of a refcompat workload: (q8 codes [T,h,576] u8,
    kv8 codes [s_kv,576] u8, q_scale, kv_scale).  Exact: q == q8*q_scale etc."""
    codes, scales, rope = split_kv_cache(kv_rows)
    if not bool((scales == REFCOMPAT_SCALE).all()):
        raise ValueError("KV cache was not generated in refcompat mode")
    q8 = e4m3_codes(q.float() / REFCOMPAT_SCALE)
    rope8 = e4m3_codes(rope.float() / REFCOMPAT_SCALE)
    kv8 = torch.cat([codes, rope8], dim=1).contiguous()
    return q8, kv8, REFCOMPAT_SCALE, REFCOMPAT_SCALE


def make_dsv4(w: Workload, seed: int = 0, device="cpu", d: int = D_QK):
    """DSv4 operands: q [T,h,d], compressed KV [Nc,d], raw KV [s_kv,d], all bf16 ~ N(0,1)."""
    gen = _gen(seed * 32452843 + 7, device)
    q = torch.randn((w.tokens, w.heads, d), generator=gen, device=device).to(torch.bfloat16)
    kc = torch.randn((w.n_compressed, d), generator=gen, device=device).to(torch.bfloat16)
    kr = torch.randn((w.s_kv, d), generator=gen, device=device).to(torch.bfloat16)
    return q, kc, kr


def dsv4_rank_space_operands(q: torch.Tensor, kv_comp: torch.Tensor, kv_raw: torch.Tensor, pos0: int,
                             heads: int, window: int, ratio: int):
    """The two-range problem in the form the reference's DSv4 operator takes it
    (kernels/b200/dsa/litedsa_dsv4.cu:40-55): a flat KV workspace [compressed | raw], one
    ascending union index list per tile (-1 padded to a multiple of 64) and the per-token
    bounds (prefix, window start, window end) in union-rank space.

    q [T,h,d], kv_comp [Nc,d], kv_raw [S,d] (any width d) -> (q [ng,128,d], kv [Nc+S,1,d],
    indices [ng,1,topk] i32, pref / win_lo / win_hi [ng,G] i32, counts [ng] i32)."""
    T, _, d = q.shape
    G = 128 // heads
    ng = T // G
    nc_all = kv_comp.shape[0]
    dev = q.device
    p_first = pos0 + torch.arange(ng, device=dev, dtype=torch.int64) * G           # [ng]
    p_tok = p_first[:, None] + torch.arange(G, device=dev, dtype=torch.int64)       # [ng, G]
    ncmax = torch.clamp(p_tok[:, -1] // ratio, max=nc_all)                           # [ng]
    lo = torch.clamp(p_first - window + 1, min=0)                                    # [ng]
    n_win = p_tok[:, -1] + 1 - lo                                                    # [ng]
    counts = (ncmax + n_win).to(torch.int32)
    topk = int((int(counts.max().item()) + 63) // 64 * 64)
    r = torch.arange(topk, device=dev, dtype=torch.int64)[None, :]                   # rank
    is_c = r < ncmax[:, None]
    widx = nc_all + lo[:, None] + (r - ncmax[:, None])
    indices = torch.where(is_c, r, torch.where(r < counts[:, None].long(), widx, torch.full_like(widx, -1)))
    pref = torch.clamp(p_tok // ratio, max=nc_all)
    win_lo = ncmax[:, None] + (torch.clamp(p_tok - window + 1, min=0) - lo[:, None])
    win_hi = ncmax[:, None] + (p_tok + 1 - lo[:, None])
    kv = torch.cat([kv_comp, kv_raw], dim=0).contiguous().view(-1, 1, d)
    return (q.contiguous().view(ng, 128, d), kv, indices.to(torch.int32).view(ng, 1, topk).contiguous(),
            pref.to(torch.int32).contiguous(), win_lo.to(torch.int32).contiguous(),
            win_hi.to(torch.int32).contiguous(), counts.contiguous())


def attended_pairs(w: Workload, topk_idx: Optional[torch.Tensor] = None) -> int:
    """Attended (query-head, key) pairs: the unit effective FLOPs are counted on."""
    if w.kind == "dsv4":
        p = torch.arange(w.pos0, w.pos0 + w.tokens, dtype=torch.int64)
        return int((w.heads * (p // w.ratio + torch.clamp(p + 1, max=w.window))).sum().item())
    if topk_idx is None:
        return w.tokens * w.heads * w.topk
    return int((topk_idx >= 0).sum().item()) * w.heads


FLOP_PER_PAIR = 2 * D_QK + 2 * D_LATENT  # QK over 576 dims + PV over 512 dims
SM_SCALE = 1.0 / math.sqrt(192.0)


def make_indexer_operands(tokens: int, s_kv: int, index_heads: int = 64, seed: int = 0, device="cpu"):
    """Synthetic operands of the FP8 lightning indexer: ``q_idx8`` [tokens, Hi, 128] and
    ``k_idx8`` [s_kv, 128] e4m3 codes (uint8) of N(0,1) values scaled to the e4m3 range,
    ``weights`` [tokens, Hi] fp32 (head weights ~ N(0,1) / sqrt(Hi) times the query scales and
    the softmax scale 128^-0.5), ``k_scale`` [s_kv] fp32 (amax / 448 per key)."""
    gen = _gen(seed * 7919 + 11, device)
    q = torch.randn((tokens, index_heads, 128), generator=gen, device=device)
    k = torch.randn((s_kv, 128), generator=gen, device=device)
    hw = torch.randn((tokens, index_heads), generator=gen, device=device) / index_heads ** 0.5
    q_scale = q.abs().amax(dim=2).clamp_min(1e-8) / E4M3_MAX            # [tokens, Hi]
    k_scale = k.abs().amax(dim=1).clamp_min(1e-8) / E4M3_MAX            # [s_kv]
    q8 = e4m3_codes(q / q_scale[:, :, None])
    k8 = e4m3_codes(k / k_scale[:, None])
    weights = (hw * q_scale * 128 ** -0.5).float().contiguous()
    return q8, k8, weights, k_scale.float().contiguous()

