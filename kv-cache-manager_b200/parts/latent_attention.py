"""Attention over a cached latent: per position one normalised vector c [rank] is kept, and every
head's keys and values are linear in it, k = W_uk c and v = W_uv c.  No position encoding.

    q = W_q h;   c = w * (W_dkv h) / rms(W_dkv h);   score_ij = scale * q_i . k_j  (j <= i);
    out = W_o concat_heads( softmax(score) v )

Only c is cached, in pages laid out like a key pool with ONE shared head of ``rank`` elements and
no value pool.  The products with W_uk and W_uv are moved across the softmax, which changes
nothing in exact arithmetic: score = (W_uk^T q) . c and sum_j p_j W_uv c_j = W_uv (sum_j p_j c_j).
So every head's query is mapped into the latent space, the engine's paged attention kernels run
with all heads sharing the latent pages as keys AND values (prefill and decode alike, portions
reading earlier portions' latents from the pages), and the head outputs are mapped back by W_uv.
A site built with ``own_latent=False`` has no W_dkv: the run order points it at an earlier site's
pages (``LayerCall.cache_of``), which it reads with its own W_uk, W_uv and queries.
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import CacheSpec, MIXERS, Mixer, SiteCache, StepContext
from .linear import Linear

BMM_MIN_ROWS = 64       # from here on the library's batched product does the per-head maps of bfloat16 rows


def per_head_product(x: torch.Tensor, w: torch.Tensor, ctx: StepContext) -> torch.Tensor:
    """x [M, B, K] (a view; K dense), w [B, N, K] -> [M, B * N]: y[m, b] = w[b] x[m, b]."""
    M, B, _ = x.shape
    N = w.shape[1]
    y = torch.empty((M, B, N), dtype=x.dtype, device=x.device)
    if x.dtype == torch.bfloat16 and M >= BMM_MIN_ROWS and ctx.options.get("gemm", "auto") in ("auto", "library"):
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=y.transpose(0, 1))
        K.profile_mark("library_gemm")
    else:
        K.gemm_plain_batched(x, w, y)
    return y.view(M, B * N)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden: int, heads: int, dk: int, dv: int, rank: int, scale: float, norm_eps: float,
                 own_latent: bool = True) -> None:
        super().__init__()
        self.hidden, self.heads, self.dk, self.dv, self.rank = hidden, heads, dk, dv, rank
        self.scale, self.norm_eps, self.own_latent = float(scale), float(norm_eps), bool(own_latent)
        std = hidden ** -0.5
        # one product for q | (latent before its norm)
        self.q_dkv = self.add_child("q_dkv", Linear(hidden, heads * dk + (rank if own_latent else 0), std))
        self.uk = self.add_child("uk", Linear(rank, heads * dk, rank ** -0.5))
        self.uv = self.add_child("uv", Linear(rank, heads * dv, rank ** -0.5))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        if own_latent:
            self.declare("latent_norm", (rank,), ("ones",), "vector")
        self._uk_t = self._uv = self._norm = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, self.rank, 0, values=False)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        H, R = self.heads, self.rank
        # W_uk [H*dk, R] as H maps from a head's query to the latent space: [H, R, dk]
        self._uk_t = self.uk.param("weight").view(H, self.dk, R).transpose(1, 2).contiguous()
        self._uv = self.uv.param("weight").view(H, self.dv, R)
        if self.own_latent:
            self._norm = self.param("latent_norm").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        M, H, R = h.shape[0], self.heads, self.rank
        proj = self.q_dkv.forward(h, ctx)
        if self.own_latent:
            if not site.writes:
                raise RuntimeError("latent_attention: a site with a latent of its own must own its pages")
            K.latent_norm_cache(proj[:, H * self.dk:], self._norm, g.slot_mapping, site.k, self.norm_eps)
        q_lat = per_head_product(proj[:, :H * self.dk].unflatten(1, (H, self.dk)), self._uk_t.to(proj.dtype), ctx)
        out_lat = torch.empty((M, H * R), dtype=h.dtype, device=h.device)
        pages = site.k
        if (h.dtype == torch.bfloat16 and ctx.options.get("attention", "auto") != "plain"
                and K.fast_attention_supported(H, 1, R, pages.shape[2]) and (H * R) % 8 == 0):
            K.paged_attention(q_lat, out_lat, pages, pages, g.block_tables, ctx, H, 1, R, self.scale, 0)
        else:
            K.attention_plain(q_lat, out_lat, pages, pages, g.block_tables, ctx.row_seq, ctx.positions, H, 1, R,
                              self.scale, 0)
        heads_out = per_head_product(out_lat.view(M, H, R), self._uv.to(out_lat.dtype), ctx)
        return self.o.forward(heads_out, ctx, out_dtype=torch.float32)
