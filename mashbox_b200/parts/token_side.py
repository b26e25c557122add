"""A per-layer input that depends on the token itself: every layer has its own stretch of a second embedding table.

    e = table[token, offset : offset + dim];   y = Wp (gelu_tanh(Wg x) * e);   x <- x + y / sqrt(mean(y^2) + eps) * w

x is the residual stream itself (not a normed copy).  The two products are ordinary products; the gather and the gate
are one kernel; the norm of y and the add into the stream are the kernel a block uses for every normed sublayer output
(`post_norm_add`), which can also leave the next norm's output.
"""
from ..weights.loader import Want
from .base import register


class GatedTokenSide:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, hidden, dim, offset, table_width, vocab, eps, prefix="", table="side.embed", names=None):
        self.D, self.dim, self.offset, self.table_width, self.V = int(hidden), int(dim), int(offset), int(table_width), int(vocab)
        self.eps, self.table_name = float(eps), table
        n = dict(gate="side.gate", proj="side.proj", norm="side.norm")
        n.update(names or {})
        self.n = {k: prefix + v for k, v in n.items()}
        self.table = self.wg = self.wp = self.norm_w = None

    def wants(self):
        return [Want(self.table_name, (self.V, self.table_width), "matrix"), Want(self.n["gate"], (self.dim, self.D), "matrix"),
                Want(self.n["proj"], (self.D, self.dim), "matrix"), Want(self.n["norm"], (self.D,), "vector")]

    def bind(self, tensors, env):
        self.table = tensors[self.table_name]
        self.wg, self.wp, self.norm_w = tensors[self.n["gate"]], tensors[self.n["proj"]], tensors[self.n["norm"]]

    def forward(self, ctx, x, xa, next_norm=None, normed=None):
        """x (N, D) the float32 stream, xa the same rows in the activation dtype (x itself on the 32-bit path).
        next_norm, normed: the norm that reads the stream next and the buffer for its output"""
        ops, N = ctx.ops, ctx.N
        z = ctx.ws.get("side_gate", N, (self.dim,), ctx.dtype)
        ops.linear(xa, self.wg, out=z)
        g = ctx.ws.get("side_act", N, (self.dim,), ctx.dtype)
        ops.gated_gather(z, ctx.dev("token_ids"), self.table, self.offset, g, ctx.err)
        y = ctx.ws.get("delta", N, (self.D,), ctx.dtype)
        ops.linear(g, self.wp, out=y)
        if next_norm is not None:
            ops.post_norm_add(x, y, self.norm_w, self.eps, next_norm.weight, next_norm.eps, normed)
        else:
            ops.post_norm_add(x, y, self.norm_w, self.eps)


register("side", "gated_table", GatedTokenSide)
