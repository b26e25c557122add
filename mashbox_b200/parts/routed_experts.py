"""A feed-forward of many small experts of which every token uses a few, chosen by a router.

    z = Wr h (float32);  s = sigmoid(z);  c = s + correction
    the experts form `groups` equal runs of neighbours; a run is worth the sum of its two largest c; experts outside the
    `keep` best runs cannot be chosen; the `top` largest c are chosen; out = sum over the chosen of s_e expert_e(h)
    expert: g = min(Wg h, limit);  u = clamp(Wu h, -limit, limit);  Wd (g sigmoid(alpha g) (u + 1))

The correction moves the choice only: the weights are the plain scores, not renormalised.  The stored matrices of the
experts (`e0`, `e1`, ...) are stacked at load into (experts, rows, columns) tensors.  A step: the router's product with
a float32 result, one kernel that chooses (a warp per token), the experts, and one kernel that sums a token's places in
order.  The experts of a step of few tokens (and of every float32 step) are one kernel with a block per (token, chosen
expert) pair that streams that expert's three matrices; a bfloat16 step of more tokens sorts the pairs by expert on
the device and runs every expert's rows through tensor-core tiles (gate and up with the activation in the epilogue,
then down), so an expert's matrices are read once per 64 of its rows.  The choice is made on
the device and every launch has a shape that follows from the number of tokens, so steps can be captured in graphs.
"""
from ..errors import ConfigError
from ..weights.loader import Want
from .base import register


class RoutedExperts:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, intermediate, experts, top, limit, groups=1, keep=1, alpha=1.702, correction=True,
                 prefix="", names=None):
        self.D, self.F, self.E, self.top = int(hidden), int(intermediate), int(experts), int(top)
        self.groups, self.keep = int(groups or 1), int(keep or 1)
        self.limit, self.alpha, self.has_correction = float(limit), float(alpha), bool(correction)
        if self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ConfigError(f"{experts} experts do not form {groups} equal groups of which {keep} are kept")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ConfigError(f"{top} experts cannot be chosen from {keep} groups of {self.E // self.groups}")
        n = dict(router="mlp.router", correction="mlp.correction", expert="mlp.e{}.", gate="gate", up="up", down="down")
        n.update(names or {})
        self.n = {k: (v if k in ("gate", "up", "down") else prefix + v) for k, v in n.items()}
        self.wr = self.corr = self.wg = self.wu = self.wd = None

    def _expert(self, e, which):
        return self.n["expert"].format(e) + self.n[which]

    def wants(self):
        out = [Want(self.n["router"], (self.E, self.D), "matrix")]
        if self.has_correction:
            out.append(Want(self.n["correction"], (self.E,), "vector"))
        for e in range(self.E):
            out += [Want(self._expert(e, "gate"), (self.F, self.D), "matrix"),
                    Want(self._expert(e, "up"), (self.F, self.D), "matrix"),
                    Want(self._expert(e, "down"), (self.D, self.F), "matrix")]
        return out

    def bind(self, tensors, env):
        import torch
        self.wr = tensors[self.n["router"]]
        self.corr = tensors[self.n["correction"]] if self.has_correction else None
        stack = lambda which: torch.stack([tensors[self._expert(e, which)] for e in range(self.E)], 0).contiguous()
        # (E, 2F, D): every expert's gate rows, then its up rows; the kernels that want them apart take views
        self.wgu = torch.cat([stack("gate"), stack("up")], 1).contiguous()
        self.wg, self.wu, self.wd = self.wgu[:, :self.F], self.wgu[:, self.F:], stack("down")

    def forward(self, ctx, h, out="delta"):
        import torch
        ops, N = ctx.ops, ctx.N
        z = ctx.ws.get("router_logits", N, (self.E,), torch.float32)
        ops.linear(h, self.wr, out=z, out_dtype=torch.float32)
        ids = ctx.ws.get("router_ids", N, (self.top,), torch.int32)
        wts = ctx.ws.get("router_weights", N, (self.top,), torch.float32)
        ops.moe_select(z, self.corr, ids, wts, self.groups, self.keep)
        if ops.moe_tc5_supports(N, self.D, self.F, ctx.dtype) and not ctx.options.get("plain_experts", False):
            T = ops.moe_tc5_tiles(ctx.ws.max_rows, self.top, self.E)
            rows = ctx.ws.get("expert_rows", 128 * T, (self.D,), ctx.dtype, reserve=128 * T)
            act = ctx.ws.get("expert_rows_act", 128 * T, (self.F,), ctx.dtype, reserve=128 * T)
            y = ctx.ws.get("expert_rows_out", 128 * T, (self.D,), torch.float32, reserve=128 * T)
            scratch = ctx.ws.get("expert_places", ctx.ws.max_rows * self.top + T, (), torch.int32,
                                 reserve=ctx.ws.max_rows * self.top + T)
            delta = ctx.ws.get(out, N, (self.D,), ctx.dtype)
            ops.moe_tc5(h, ids, wts, self.wgu, self.wd, delta, rows, act, y, scratch, self.limit, self.alpha)
            return delta, None
        y = ctx.ws.get("expert_out", N, (self.top, self.D), torch.float32)
        if ops.moe_grouped_supports(N, self.D, self.F, ctx.dtype) and not ctx.options.get("plain_experts", False):
            act = ctx.ws.get("expert_act", N * self.top, (self.F,), ctx.dtype, reserve=ctx.ws.max_rows * self.top)
            n = ops.moe_grouped_scratch(ctx.ws.max_rows, self.top, self.E)
            scratch = ctx.ws.get("expert_sort", max(n, ops.moe_grouped_scratch(N, self.top, self.E)), (), torch.int32, reserve=n)
            ops.moe_grouped(h, ids, self.wg, self.wu, self.wd, y, act, scratch, self.limit, self.alpha)
        else:
            # bfloat16 steps of many tokens take the other form: room for the few
            most = min(ctx.ws.max_rows, max(N, ops.MOE_GROUPED["tokens"])) if ctx.dtype == torch.bfloat16 else ctx.ws.max_rows
            act = ctx.ws.get("expert_act_few", N * self.top, (self.F,), torch.float32, reserve=most * self.top)
            ops.moe_experts(h, ids, self.wg, self.wu, self.wd, y, self.limit, self.alpha, act)
        delta = ctx.ws.get(out, N, (self.D,), ctx.dtype)
        ops.moe_combine(y, wts, delta)
        return delta, None


register("feed_forward", "routed_experts", RoutedExperts)
