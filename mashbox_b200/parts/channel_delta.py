"""The channel-wise gated delta rule mixer: a recurrent layer whose state is a matrix per head, decayed per key channel.

    q, k = silu(conv(Wq h)), silu(conv(Wk h))  (kv_heads x dim; head h reads q/k head h // (heads / kv_heads))
    v    = silu(conv(Wv h))                    (heads x vdim)
    q, k to unit vectors per head, x / sqrt(sum x^2 + 1e-6); q also times dim^-1/2
    beta = sigmoid(Wb h)                       (one per head)
    g    = exp(-exp(A_h) softplus(Wa2 (Wa1 h) + dt_bias))      (heads x dim, one decay per head and key channel)
    per head and token:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out  = Wo concat_h (o_h / sqrt(mean(o_h^2) + eps) * n * sigmoid(Wg2 (Wg1 h))_h)

conv is a short causal convolution over time per channel (`taps`; None: none).  The layer keeps nothing per position;
per request it keeps one flat float32 state: the last taps - 1 rows of the q/k/v product (what the convolutions need of
the past), then S (heads, dim, vdim).  A state slot is zeroed when a request takes it, which is both "zeros before
the start" and "the state starts at zero".

A step: three products of the mixer's input (q/k/v rows; the narrow rows beta, Wa1, Wg1; then the two wide rows from
the narrow ones with Wa2 and Wg2 side by side in one block-diagonal matrix), the convolution kernel, one kernel that
makes everything the recurrence reads in float32, the recurrence (a sequence's tokens in order, whatever their number:
prompts, portions and single tokens are one loop), the gated norm of its output, the output product.  Decays, their
logarithms, softplus, beta, the unit norms, the state and the recurrence are float32.
"""
from ..cache.manager import StateNeed
from ..errors import ConfigError
from ..weights.loader import Want
from .base import register
from .conv import plan_sequences, state_view, step_sequences


class ChannelDelta:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, heads, kv_heads, dim, vdim, eps, taps=None, decay_rank=None, gate_rank=None, unit_eps=1e-6,
                 prefix="", names=None):
        self.D, self.H, self.G, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        if self.G < 1 or self.H % self.G:
            raise ConfigError(f"{heads} heads do not divide into {kv_heads} kv heads")
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.has_conv = bool(taps)              # None or 0: no convolution; 1: a filter of one tap, which keeps no state
        self.taps = int(taps) if taps else 1
        # the inner widths of the two low-rank products; None: whatever the stored tensors have
        self.decay_rank = int(decay_rank) if decay_rank else -1
        self.gate_rank = int(gate_rank) if gate_rank else -1
        n = dict(q="q", k="k", v="v", conv=".conv", b="b", A="A_log", norm="norm", a1="a1", a2="a2", dt="dt_bias", g1="g1",
                 g2="g2", o="o")
        n.update(names or {})
        self.n = {k: (v if k == "conv" else prefix + v) for k, v in n.items()}
        self.rows = dict(q=self.G * self.dim, k=self.G * self.dim, v=self.H * self.vdim)
        self.C = sum(self.rows.values())
        self.state_offset = 0
        self.w_qkv = self.w_low = self.w_wide = self.wconv = self.wo = self.A = self.dt = self.norm_w = None

    def wants(self):
        D, H = self.D, self.H
        out = []
        for r in "qkv":
            out.append(Want(self.n[r], (self.rows[r], D), "matrix"))
            if self.has_conv:
                out.append(Want(self.n[r] + self.n["conv"], (self.rows[r], self.taps), "vector"))
        out += [Want(self.n["b"], (H, D), "matrix"), Want(self.n["A"], (H,), "vector"),
                Want(self.n["norm"], (self.vdim,), "vector"), Want(self.n["a1"], (self.decay_rank, D), "matrix"),
                Want(self.n["a2"], (H * self.dim, self.decay_rank), "matrix"), Want(self.n["dt"], (H * self.dim,), "vector"),
                Want(self.n["g1"], (self.gate_rank, D), "matrix"), Want(self.n["g2"], (H * self.vdim, self.gate_rank), "matrix"),
                Want(self.n["o"], (D, H * self.vdim), "matrix")]
        return out

    def bind(self, tensors, env):
        import torch
        t = lambda k: tensors[self.n[k]]
        a1, a2, g1, g2 = t("a1"), t("a2"), t("g1"), t("g2")
        if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
            raise ConfigError("the two matrices of a low-rank product do not fit each other")
        ra, rg, H = a1.shape[0], g1.shape[0], self.H
        self.w_qkv = torch.cat([t("q"), t("k"), t("v")], 0).contiguous()
        self.w_low = torch.cat([t("b"), a1, g1], 0).contiguous()               # narrow rows: [beta | decay | gate]
        wide = torch.zeros((H * self.dim + H * self.vdim, H + ra + rg), dtype=a2.dtype, device=a2.device)
        wide[:H * self.dim, H:H + ra] = a2                                      # zeros elsewhere: exact in any dtype
        wide[H * self.dim:, H + ra:] = g2
        self.w_wide = wide
        self.wconv = (torch.cat([tensors[self.n[r] + self.n["conv"]] for r in "qkv"], 0).t().contiguous()
                      if self.has_conv else None)                               # (taps, channels)
        self.A, self.dt, self.norm_w, self.wo = t("A"), t("dt"), t("norm"), t("o")

    def cache_need(self):
        return None

    def conv_floats(self):
        return (self.taps - 1) * self.C

    def state_floats(self):
        return self.conv_floats() + self.H * self.dim * self.vdim

    def state_need(self):
        return StateNeed((self.state_floats(),), "float32")

    def prepare(self, ctx):
        plan_sequences(ctx)

    def forward(self, ctx, h, run):
        import torch
        ops, N = ctx.ops, ctx.N
        H, G, dim, vdim = self.H, self.G, self.dim, self.vdim
        qkv = ctx.ws.get("delta_qkv", N, (self.C,), ctx.dtype)
        ops.linear(h, self.w_qkv, out=qkv)
        low = ctx.ws.get("delta_low", N, (self.w_low.shape[0],), ctx.dtype)
        ops.linear(h, self.w_low, out=low)
        wide = ctx.ws.get("delta_wide", N, (self.w_wide.shape[0],), ctx.dtype)
        ops.linear(low, self.w_wide, out=wide)
        if self.has_conv:
            conv = ctx.ws.get("delta_conv", N, (self.C,), ctx.dtype)
            ops.short_conv(qkv, self.wconv, state_view(ctx, run.state_id, self.state_offset, self.taps, self.C),
                           step_sequences(ctx), conv)
            qkv = conv
        f32 = torch.float32
        q = ctx.ws.get("delta_q", N, (G * dim,), f32)
        k = ctx.ws.get("delta_k", N, (G * dim,), f32)
        v = ctx.ws.get("delta_v", N, (H * vdim,), f32)
        g = ctx.ws.get("delta_g", N, (H * dim,), f32)
        beta = ctx.ws.get("delta_beta", N, (H,), f32)
        ops.delta_gates(qkv, low, wide, self.A, self.dt, q, k, v, g, beta, H, G, dim, vdim, self.unit_eps)
        o = ctx.ws.get("delta_o", N, (H * vdim,), f32)
        off = self.state_offset + self.conv_floats()
        state = ctx.cache.state[run.state_id][:, off:off + H * dim * vdim]
        ops.delta_rule(q, k, v, g, beta, o, state, (ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("state_slot")), H, G,
                       dim, vdim)
        out = ctx.ws.get("attn_out", N, (H * vdim,), ctx.dtype)
        ops.gated_rms(o, wide[:, H * dim:], self.norm_w, out, H, vdim, self.eps)
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(out, self.wo, out=y)
        return y, None


register("mixer", "channel_delta", ChannelDelta)
