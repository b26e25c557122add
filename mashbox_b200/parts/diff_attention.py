"""The differential attention mixer: two softmax attention maps per head over one set of values, their difference
normalised per head.

Every head has two maps with queries and keys of their own (rows of the q and k projections lie head by head as
[map 0 | map 1], `dim` each) and shares its values (`vdim` wide) between them:

    a_m = softmax(scale q_m K_m^T) V,    o = a_0 - lam a_1,    out = o / sqrt(mean(o^2) + eps) * (1 - delta)

with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + delta, one number for the layer, made at load in float64 from its four
vectors.  Query head h reads kv head h // (H / G).  Options, each a constructor parameter: biases on q/k/v; a short
causal convolution over time on every channel of q, k and v right after the projection (`taps`; the last taps - 1
projected rows are carried in the layer's state); a rotation of the first dims of every map (`position`, a rotary
encoding with the halves pairing); `chunk`: a query sees the keys of its own block of `chunk` positions, counted from
the sequence's start, up to itself (None: all earlier keys); `shares_kv`: the layer has no k/v projections and reads
the cache another layer wrote (its schedule entry names that cache), with its own queries and mask.

A step: one fused q/k/v product; one kernel adds the biases, convolves, rotates, stores the keys (both maps of a kv
head side by side) and values in their pages and the queries in a buffer; the attention kernel reads the step's own
tokens from the cache like older ones, so whole prompts, portions and single tokens take one path; then the output
product.  Scores, softmaxes, weighted sums, the difference and the head norm are float32.
"""
import math

import numpy as np

from ..cache.manager import CacheNeed, StateNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import PartSpec, make, register
from .conv import plan_sequences, state_view, step_sequences


def plan_diff_tiles(q_len, pos0, group, rows):
    """Work list of the prompt form of the tensor-core kernel: one (sequence, tile) pair per `rows` packed query rows --
    a sequence's tokens times the `group` query heads of a kv head -- the tiles that reach the most keys first.
    -> flat int list"""
    return plan_diff_attention(q_len, pos0, group, 1, None, rows, decode_rows=0)["pre"]


def plan_diff_attention(q_len, pos0, group, kv_heads, chunk, rows, decode_rows=16, max_splits=16, target=296, splits=None,
                        quads=False):
    """The two work lists of the tensor-core kernels of the differential attention, as flat int lists.  "pre": (sequence,
    tile of `rows` packed rows) for sequences of more than `decode_rows` packed rows (`quads`: as (sequence, tile, 0,
    1), the form the tcgen05 kernel reads).  "dec": (sequence, split, number
    of splits, slot) for the others: their keys -- from the start of the block of `chunk` positions the sequence's first
    query lies in -- are cut into a power of two of splits, as many as fill `target` blocks with the step's decode-form
    sequences times the kv heads, never fewer than two tiles of 64 keys to a split (`splits`: that many, whatever the
    sizes).  "slots": (sequence, number of splits) of the sequences that are cut; the kernel that merges the splits runs
    over these."""
    pre, dec, slots = [], [], []
    short = [s for s, n in enumerate(q_len) if n * group <= decode_rows]
    want = max(1, target // max(1, len(short) * kv_heads))
    for s, n in enumerate(q_len):
        if n * group > decode_rows:
            for m in range(-(-n * group // rows)):
                pre.append((-(pos0[s] + min(n, (m + 1) * rows // group)), s, m))
            continue
        lo = pos0[s] // chunk * chunk if chunk else 0
        tiles = -(-(pos0[s] + n - lo // 64 * 64) // 64)
        ns = max(1, min(max_splits, want, tiles // 2)) if splits is None else max(1, min(max_splits, int(splits)))
        ns = 1 << (ns.bit_length() - 1)
        slot = -1
        if ns > 1:
            slot = len(slots)
            slots.append((s, ns))
        dec += [(s, sp, ns, slot) for sp in range(ns)]
    pre.sort()
    flat = lambda items: [v for it in items for v in it]
    return dict(pre=flat([it[1:] + ((0, 1) if quads else ()) for it in pre]), dec=flat(dec), slots=flat(slots))


class DifferentialAttention:
    @property
    def graph_safe(self):
        """forward() depends on the batch only through the lengths of the step's arrays; so must the position encoding"""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden, heads, kv_heads, dim, vdim, delta, eps, scale=None, bias=True, taps=None, position=None,
                 chunk=None, shares_kv=False, prefix="", names=None):
        self.D, self.H, self.G, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G < 1 or self.H % self.G:
            raise ConfigError(f"{heads} heads do not divide into {kv_heads} kv heads")
        self.delta, self.eps = float(delta), float(eps)
        self.scale = float(scale) if scale else self.dim ** -0.5
        self.bias = bool(bias)
        self.has_conv = bool(taps)              # taps None or 0: no convolution; 1: a filter of one tap, no state
        self.taps = int(taps) if taps else 1
        self.chunk = int(chunk) if chunk else None
        self.shares_kv = bool(shares_kv)
        n = dict(q="q", k="k", v="v", o="o", bias=".b", conv=".conv", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")
        n.update(names or {})
        self.n = {k: (v if k in ("bias", "conv") else prefix + v) for k, v in n.items()}
        self.position = make("position", position) if isinstance(position, PartSpec) else position
        self.roles = ("q",) if self.shares_kv else ("q", "k", "v")
        self.rows = dict(q=self.H * 2 * self.dim, k=self.G * 2 * self.dim, v=self.G * self.vdim)
        self.C = sum(self.rows[r] for r in self.roles)
        self.state_offset = 0
        self.w = self.b = self.wconv = self.wo = self.lam = None

    # ------------------------------------------------------------------------------------------ weights
    def wants(self):
        out = []
        for r in self.roles:
            out.append(Want(self.n[r], (self.rows[r], self.D), "matrix"))
            if self.bias:
                out.append(Want(self.n[r] + self.n["bias"], (self.rows[r],), "vector"))
            if self.has_conv:
                out.append(Want(self.n[r] + self.n["conv"], (self.rows[r], self.taps), "vector"))
        out += [Want(self.n[v], (self.dim,), "vector") for v in ("lq1", "lk1", "lq2", "lk2")]
        out.append(Want(self.n["o"], (self.D, self.H * self.vdim), "matrix"))
        return out + (self.position.wants() if self.position is not None else [])

    def bind(self, tensors, env):
        import torch
        cat = lambda suffix: torch.cat([tensors[self.n[r] + suffix] for r in self.roles], 0).contiguous()
        self.w = cat("")
        self.b = cat(self.n["bias"]) if self.bias else None
        self.wconv = cat(self.n["conv"]).t().contiguous() if self.has_conv else None      # (taps, channels)
        self.wo = tensors[self.n["o"]]
        dot = lambda a, b: float((tensors[self.n[a]].double() * tensors[self.n[b]].double()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.delta
        if self.position is not None:
            self.position.bind(tensors, env)
            rot = self.position.rotation()
            if rot is None or rot[2] != 1 or rot[1] > self.dim:
                raise ConfigError("the differential attention mixer rotates the first dims of a map, dim i with dim "
                                  "i + half: its position encoding must be rotary with the halves pairing")

    def cache_need(self):
        return CacheNeed("chunk" if self.chunk else "full", ((self.G, 2 * self.dim), (self.G, self.vdim)), self.chunk)

    def state_floats(self):
        return (self.taps - 1) * self.C

    def state_need(self):
        return StateNeed((self.state_floats(),), "float32") if self.taps > 1 else None

    def uses_mma(self, ctx):
        import torch
        return (ctx.dtype == torch.bfloat16 and ctx.ops.attention_diff_mma_supports(self.dim, self.vdim)
                and not ctx.options.get("plain_attention", False))

    def prepare(self, ctx):
        """host side: the sequences' indexes for the convolution kernels and, for the tensor-core kernel, the list of
        (sequence, row tile) work items (one list for all layers with the same number of query heads per kv head)"""
        plan_sequences(ctx)
        if not self.uses_mma(ctx):
            return
        key = self.plan_key()
        if key not in ctx.memo:
            name = "diff%d_" % len([k for k in ctx.memo if k[0] == "diff_attention"])
            tc5 = self.uses_tc5(ctx)
            rows = ctx.ops.attention_tc5_diff_rows() if tc5 else ctx.ops.attention_diff_mma_rows()
            plan = plan_diff_attention(ctx.q_len, ctx.pos0, self.H // self.G, self.G, self.chunk, rows,
                                       ctx.ops.DIFF_DECODE_ROWS, ctx.ops.DIFF_MAX_SPLITS,
                                       int(ctx.options.get("attention_target_blocks", 296)),
                                       ctx.options.get("attention_splits"), quads=tc5)
            for k, v in plan.items():
                ctx.inputs.add(name + k, np.asarray(v, np.int32))
            ctx.memo[key] = dict(name=name, tc5=tc5, n_pre=len(plan["pre"]) // (4 if tc5 else 2),
                                 n_dec=len(plan["dec"]) // 4, n_slots=len(plan["slots"]) // 2)

    def uses_tc5(self, ctx):
        """prompt-form tiles go to the tcgen05 kernel when a row of two maps is as wide as a value row of 64 or 128"""
        return (ctx.options.get("attention_prefill_kernel", "tc5") == "tc5"
                and ctx.ops.attention_tc5_diff_supports(self.dim, self.vdim, ctx.cache.page_size))

    def plan_key(self):
        # everything the work lists depend on (the head sizes decide the kernel and its rows per tile)
        return ("diff_attention", self.H // self.G, self.G, self.chunk, self.dim, self.vdim)

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, ctx, h, run):
        ops, N = ctx.ops, ctx.N
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        if run.write == self.shares_kv:
            raise ConfigError("a differential attention layer writes the cache it owns and only reads one it borrows")
        qkv = ctx.ws.get("qkv", N, (self.C,), ctx.dtype)
        ops.linear(h, self.w, out=qkv)
        group, kpool, vpool = ctx.cache.layer_cache(run.cache)
        table, page, pages = group.device_table, ctx.cache.page_size, ctx.cache.pool_pages
        freqs, rd, _ = self.position.rotation() if self.position is not None else (None, 0, 1)
        q = ctx.ws.get("diff_q", N, (H * 2 * dim,), ctx.dtype)
        own = not self.shares_kv
        ops.conv_rope_kv_write(qkv, self.b, self.wconv, state_view(ctx, run.state_id, self.state_offset, self.taps, self.C),
                               step_sequences(ctx), ctx.dev("positions"), ctx.dev("tok_row"), table, q,
                               kpool if own else None, vpool if own else None, freqs, 2 * H, 2 * G if own else 0,
                               G if own else 0, dim, vdim, 2, rd, page, pages, ctx.err)
        out = ctx.ws.get("attn_out", N, (H * vdim,), ctx.dtype)
        if self.uses_mma(ctx):
            import torch
            plan = ctx.memo[self.plan_key()]
            nm = plan["name"]
            seqs = (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("pos0"), ctx.dev("seq_row"))
            tail = (table, kpool, vpool, H, G, dim, vdim, page, pages, self.chunk, self.scale, self.lam, 1.0 - self.delta,
                    self.eps, ctx.err)
            if plan["n_pre"]:
                prompt_form = ops.attention_tc5_diff if plan["tc5"] else ops.attention_diff_mma
                prompt_form(q, out, ctx.dev(nm + "pre"), plan["n_pre"], *seqs, *tail)
            if plan["n_dec"]:
                part_o = part_ml = None
                if plan["n_slots"]:
                    n = plan["n_slots"] * G * ops.DIFF_MAX_SPLITS * 2 * ops.DIFF_DECODE_ROWS
                    part_o = ctx.ws.get("diff_part_o", n, (vdim,), torch.float32, reserve=0)
                    part_ml = ctx.ws.get("diff_part_ml", n, (2,), torch.float32, reserve=0)
                ops.attention_diff_mma_decode(q, out, ctx.dev(nm + "dec"), plan["n_dec"], ctx.dev(nm + "slots"),
                                              plan["n_slots"], part_o, part_ml, *seqs, *tail)
        else:
            ops.attention_diff_simple(q, out, ctx.dev("positions"), ctx.dev("tok_row"), table, kpool, vpool, H, G, dim,
                                      vdim, page, pages, self.chunk, self.scale, self.lam, 1.0 - self.delta, self.eps,
                                      ctx.err)
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(out, self.wo, out=y)
        return y, None


register("mixer", "differential_attention", DifferentialAttention)
