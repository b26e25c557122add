"""A short causal convolution over time with one filter per channel, carried across steps.

y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before a sequence's start; `residual` adds u_t.  What a step cannot
see -- the taps - 1 inputs before its first token -- every sequence keeps in its state slot, (taps - 1, channels)
float32, oldest first, and the kernel replaces it with the step's last inputs.  The part owns a stretch of its layer's
flat state tensor: whoever builds the layer says where it starts (`state_offset`).  Mixers that convolve their
projections use the same kernels and the same state layout through `step_sequences`.
"""
import numpy as np

from ..cache.manager import StateNeed
from ..weights.loader import Want
from .base import register


def plan_sequences(ctx):
    """host side, once per step: the index of every token's sequence among the step's sequences"""
    if not ctx.inputs.has("tok_seq"):
        ctx.inputs.add("tok_seq", np.repeat(np.arange(ctx.S, dtype=np.int32), ctx.q_len))


def step_sequences(ctx):
    """-> the four device arrays the convolution kernels tell the step's sequences apart by"""
    return ctx.dev("tok_seq"), ctx.dev("q_start"), ctx.dev("q_len"), ctx.dev("state_slot")


def state_view(ctx, state_id, offset, taps, channels):
    """the (slots, (taps - 1) * channels) stretch of a layer's flat state that one convolution owns"""
    if taps <= 1:
        return None
    return ctx.cache.state[state_id][:, offset:offset + (taps - 1) * channels]


class ShortConv:
    graph_safe = True       # forward() depends on the batch only through the lengths of the step's arrays

    def __init__(self, channels, taps, name, residual=False):
        self.C, self.taps, self.name, self.residual = int(channels), int(taps), name, bool(residual)
        self.weight, self.state_offset = None, 0

    def wants(self):
        return [Want(self.name, (self.C, self.taps), "vector")]

    def bind(self, tensors, env):
        self.weight = tensors[self.name].t().contiguous()          # tap by tap, as the kernels read them

    def state_floats(self):
        return (self.taps - 1) * self.C

    def state_need(self):
        return StateNeed((self.state_floats(),), "float32") if self.taps > 1 else None

    def prepare(self, ctx):
        plan_sequences(ctx)

    def foldable(self, ctx, state_id):
        """the kernel that makes the layer's two norms can take this convolution in for one-token stretches (it reads
        eight channels at a time, state included)"""
        if not (self.residual and self.taps > 1 and self.C % 8 == 0):
            return False
        view = state_view(ctx, state_id, self.state_offset, self.taps, self.C)
        return view.stride(0) % 4 == 0 and view.data_ptr() % 16 == 0

    def folded(self, ctx, state_id):
        """-> (filters, state view) for the norm kernel that folds the convolution in"""
        return self.weight, state_view(ctx, state_id, self.state_offset, self.taps, self.C)

    def forward(self, ctx, h, state_id, out="conv_out"):
        y = ctx.ws.get(out, h.shape[0], (self.C,), ctx.dtype)
        ctx.ops.short_conv(h, self.weight, state_view(ctx, state_id, self.state_offset, self.taps, self.C),
                           step_sequences(ctx), y, self.residual)
        return y


register("conv", "short", ShortConv)
