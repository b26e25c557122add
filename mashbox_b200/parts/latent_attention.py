"""The latent attention mixer: keys and values are projections of ONE latent vector per position, and only that vector
is kept.

    cq = rms(Wdq h) nq;   q = Wuq cq  (heads x dim)
    c  = rms(Wdkv h) nkv  (kv_rank values: the row a position keeps in its page)
    k_h = Wuk_h c,  v_h = Wuv_h c;   o_h = softmax(scale q_h K_h^T) V_h over the positions up to the query's own
    out = Wo (concat_h o_h * sigmoid(Wg h))

There is no position encoding.  Since k_h is linear in c, the score q_h . (Wuk_h c) equals (Wuk_h^T q_h) . c, and the
weighted sum of the v_h is Wuv_h applied to the weighted sum of the c: every head attends to the SAME rows -- the
latents in their pages -- with a query of kv_rank values, and its result is brought to vdim values afterwards.  That
is attention with one kv head of head size kv_rank in which a position's row is key and value at once, so the step
runs the engine's paged attention kernels (`PagedAttention`: plain, mma.sync, TMA, tcgen05 by head size) on the latent
pool, between two per-head products.  Nothing but c is ever read from the cache, whole prompts, portions and single
tokens alike.  `shares_kv`: the layer has no Wdkv and reads the latents another layer wrote (its schedule entry names
that cache), with its own Wuk, Wuv and queries.  Norms, scores, softmax and the weighted sums are float32.
"""
from ..cache.manager import CacheNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .attention import PagedAttention
from .base import register


class LatentAttention:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, heads, dim, vdim, q_rank, kv_rank, eps, scale=None, gate=True, shares_kv=False, prefix="",
                 names=None):
        self.D, self.H, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale else self.dim ** -0.5
        self.gate, self.shares_kv = bool(gate), bool(shares_kv)
        n = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        # every head's query of kv_rank values over the one row a position keeps
        self.core = PagedAttention(self.H, 1, self.kv_rank, None, self.scale)
        self.w_in = self.nq = self.nkv = self.wuq = self.wuk = self.wuv = self.wo = None

    def wants(self):
        H, D = self.H, self.D
        out = [Want(self.n["dq"], (self.q_rank, D), "matrix"), Want(self.n["dq_norm"], (self.q_rank,), "vector"),
               Want(self.n["uq"], (H * self.dim, self.q_rank), "matrix"),
               Want(self.n["uk"], (H * self.dim, self.kv_rank), "matrix"),
               Want(self.n["uv"], (H * self.vdim, self.kv_rank), "matrix"),
               Want(self.n["o"], (D, H * self.vdim), "matrix")]
        if not self.shares_kv:
            out += [Want(self.n["dkv"], (self.kv_rank, D), "matrix"), Want(self.n["dkv_norm"], (self.kv_rank,), "vector")]
        if self.gate:
            out.append(Want(self.n["g"], (H * self.vdim, D), "matrix"))
        return out

    def bind(self, tensors, env):
        import torch
        t = lambda k: tensors[self.n[k]]
        first = [t("dq")] + ([] if self.shares_kv else [t("dkv")]) + ([t("g")] if self.gate else [])
        self.w_in = torch.cat(first, 0).contiguous()           # one product: [query latent | kept latent | gate]
        self.nq = t("dq_norm")
        self.nkv = None if self.shares_kv else t("dkv_norm")
        self.wuq, self.wuk, self.wuv, self.wo = t("uq"), t("uk"), t("uv"), t("o")

    def cache_need(self):
        return CacheNeed("full", ((1, self.kv_rank),))

    def state_need(self):
        return None

    def prepare(self, ctx):
        self.core.prepare(ctx)

    def forward(self, ctx, h, run):
        ops, N, H = ctx.ops, ctx.N, self.H
        if run.write == self.shares_kv:
            raise ConfigError("a latent attention layer writes the cache it owns and only reads one it borrows")
        own = not self.shares_kv
        rows = ctx.ws.get("latent_in", N, (self.w_in.shape[0],), ctx.dtype)
        ops.linear(h, self.w_in, out=rows)
        group, pool = ctx.cache.layer_cache(run.cache)
        table, page, pages = group.device_table, ctx.cache.page_size, ctx.cache.pool_pages
        cq = ctx.ws.get("latent_q", N, (self.q_rank,), ctx.dtype)
        ops.rms_segments(rows, 0, self.nq, cq, self.q_rank, self.nkv, pool if own else None, ctx.dev("positions"),
                         ctx.dev("tok_row"), table, page, pages, self.eps, ctx.err)
        q = ctx.ws.get("latent_heads_q", N, (H * self.dim,), ctx.dtype)
        ops.linear(cq, self.wuq, out=q)
        qa = ctx.ws.get("latent_query", N, (H * self.kv_rank,), ctx.dtype)
        ops.head_product(q, self.wuk, qa, H, transposed=True)                   # Wuk_h^T q_h
        oa = ctx.ws.get("latent_mix", N, (H * self.kv_rank,), ctx.dtype)
        self.core.attend(ctx, qa, H * self.kv_rank, oa, table, pool, pool)
        o = ctx.ws.get("attn_out", N, (H * self.vdim,), ctx.dtype)
        ops.head_product(oa, self.wuv, o, H, transposed=False)                  # Wuv_h (sum of weighted latents)
        if self.gate:
            off = self.q_rank + (self.kv_rank if own else 0)
            ops.sigmoid_mul(o, rows[:, off:off + H * self.vdim])
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(o, self.wo, out=y)
        return y, None


register("mixer", "latent_attention", LatentAttention)
