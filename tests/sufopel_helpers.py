"""Small Sufopel configurations with random weights, and the plain implementation's logits for them."""
import functools
import os

import numpy as np
import torch

from mashbox_b200.config.sufopel import DeltaMixer, DenseFF, LatentMixer, RoutedFF, SufopelConfig, SufopelLayer
from tests.plain import sufopel as plain
from tests.plain.llama import read_model


def delta(heads, kv, dim, vdim, conv, ra, rg):
    return DeltaMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv, a_rank=ra, g_rank=rg)


def latent(heads, dim, vdim, q_rank, kv_rank, scale, kv_from=None):
    return LatentMixer(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, kv_from=kv_from)


# T: every size differs from layer to layer where it may.  Two query heads per kv head and key and value sizes that
#    differ in the delta layers; filters of 4 and 2 taps; experts in 3 groups of which 2 are kept with 3 chosen, and
#    ungrouped experts; a latent layer that borrows its latents, has other head sizes and no feed-forward; latents of 40
#    values (no multiple of 16: the plain attention kernel in bfloat16 too)
SUF_T = SufopelConfig("Sufopel", width=64, vocab=131, max_positions=448, embedding_scale=2.0, logit_scale=0.25,
                      norm_eps=1e-5, side_dim=8, layers=(
    SufopelLayer("channel_delta", delta(4, 2, 16, 24, 4, 8, 12), DenseFF(96)),
    SufopelLayer("latent_attention", latent(3, 16, 24, 40, 40, 0.3), RoutedFF(32, 0.7, 12, 3, 3, 2)),
    SufopelLayer("channel_delta", delta(2, 2, 24, 16, 2, 5, 4), RoutedFF(48, 1.5, 8, 2, 1, 1)),
    SufopelLayer("latent_attention", latent(2, 8, 16, 24, 40, 0.5, kv_from=1), None)))
# U: what T does not have: no token input, scales of 1, one kv head, a delta layer without filters and one with filters
#    of ONE tap (they keep no state), one chosen expert, every expert a group of its own, a latent layer first
SUF_U = SufopelConfig("Sufopel", width=96, vocab=89, max_positions=512, embedding_scale=1.0, logit_scale=1.0,
                      norm_eps=1e-6, side_dim=None, layers=(
    SufopelLayer("latent_attention", latent(4, 24, 8, 16, 32, 0.25), DenseFF(64)),
    SufopelLayer("channel_delta", delta(3, 1, 40, 20, None, 6, 6), RoutedFF(24, 1.0, 6, 1, 6, 2)),
    SufopelLayer("channel_delta", delta(2, 1, 8, 72, 1, 3, 9), None),
    SufopelLayer("latent_attention", latent(4, 24, 8, 16, 32, 0.2, kv_from=0), DenseFF(40))))
# V: sizes the tensor-core kernels take: latents of 64 and of 128 values, 8 heads (their rows packed into one tile),
#    delta heads of 64 x 32
SUF_V = SufopelConfig("Sufopel", width=128, vocab=301, max_positions=640, embedding_scale=0.5, logit_scale=2.0,
                      norm_eps=2e-6, side_dim=16, layers=(
    SufopelLayer("latent_attention", latent(8, 16, 16, 48, 64, 0.25), RoutedFF(64, 2.0, 16, 4, 4, 2)),
    SufopelLayer("channel_delta", delta(4, 4, 64, 32, 3, 16, 8), DenseFF(192)),
    SufopelLayer("latent_attention", latent(4, 32, 32, 64, 128, 0.18), DenseFF(96)),
    SufopelLayer("latent_attention", latent(8, 16, 32, 32, 64, 0.25, kv_from=0), RoutedFF(32, 0.5, 4, 2, 2, 1))))
# W: delta layers only -- the model keeps nothing per position, the cache manager has no group and no page is ever taken
SUF_W = SufopelConfig("Sufopel", width=48, vocab=61, max_positions=448, embedding_scale=1.5, logit_scale=0.5,
                      norm_eps=1e-5, side_dim=4, layers=(
    SufopelLayer("channel_delta", delta(2, 1, 16, 8, 3, 4, 4), DenseFF(64)),
    SufopelLayer("channel_delta", delta(1, 1, 32, 48, 2, 8, 2), RoutedFF(16, 1.2, 4, 2, 2, 2))))
# X: latent layers only (no state), latents of 288 values: wider than any tensor-core attention kernel takes
SUF_X = SufopelConfig("Sufopel", width=80, vocab=73, max_positions=448, embedding_scale=1.0, logit_scale=1.0,
                      norm_eps=1e-6, side_dim=None, layers=(
    SufopelLayer("latent_attention", latent(2, 24, 40, 32, 288, 0.2), DenseFF(96)),
    SufopelLayer("latent_attention", latent(5, 8, 8, 16, 288, 0.35, kv_from=0), None)))
# Y: more heads than a decode tile of the tensor-core attention kernels has rows (20 and 24 over one row per position):
#    a single decoded token is a prompt-form tile, which the plan cuts along the keys
SUF_Y = SufopelConfig("Sufopel", width=64, vocab=97, max_positions=448, embedding_scale=1.0, logit_scale=1.5,
                      norm_eps=1e-5, side_dim=None, layers=(
    SufopelLayer("latent_attention", latent(20, 8, 8, 32, 64, 0.3), DenseFF(64)),
    SufopelLayer("channel_delta", delta(2, 2, 16, 16, 2, 4, 4), None),
    SufopelLayer("latent_attention", latent(24, 8, 4, 16, 64, 0.25, kv_from=0), DenseFF(48))))
# Z: sizes that are multiples of neither 8 nor 16, so that no 16-byte form of any kernel applies: width 100, heads of
#    12 x 20 and 10 x 6, latents of 28 from a query latent of 20, experts of 28, a token input of 6, a page of 5 positions
SUF_Z = SufopelConfig("Sufopel", width=100, vocab=53, max_positions=448, embedding_scale=0.75, logit_scale=1.25,
                      norm_eps=1e-5, side_dim=6, layers=(
    SufopelLayer("channel_delta", delta(3, 3, 12, 20, 3, 5, 7), RoutedFF(28, 0.9, 6, 2, 3, 2)),
    SufopelLayer("latent_attention", latent(3, 10, 6, 20, 28, 0.3), DenseFF(44)),
    SufopelLayer("channel_delta", delta(2, 1, 10, 6, 5, 3, 3), None),
    SufopelLayer("latent_attention", latent(5, 6, 10, 12, 28, 0.4, kv_from=1), RoutedFF(12, 2.0, 5, 3, 1, 1))))
CONFIGS = {"T": (SUF_T, 11, 8), "U": (SUF_U, 12, 16), "V": (SUF_V, 13, 16), "W": (SUF_W, 14, 32),
           "X": (SUF_X, 15, 8), "Y": (SUF_Y, 16, 16), "Z": (SUF_Z, 17, 5)}       # config, seed, page size

# Readers near 1/sqrt(fan in), writers into the stream small; filters, decays and corrections of order 0.3 to 1 so
# that they matter; the router wide enough that the chosen experts are seldom a close call.
STD_BY_NAME = ((".conv", 0.4), ("A_log", 0.5), ("dt_bias", 1.0), ("correction", 0.2), ("mlp.router", 0.4), (".ls", 0.3),
               ("mix.o", 0.05), ("mlp.down", 0.05), (".down", 0.1), ("side.proj", 0.05), ("embed", 0.5), ("pos", 0.3),
               ("mix.a2", 0.5), ("mix.g2", 0.5), ("mix.uk", 0.3), ("mix.uq", 0.3))


# A sublayer's output is normed before it joins the stream, so which experts a token gets moves its row by a fixed,
# large amount however small the experts' weights are, and the recurrent state and the latents carry that to every
# later row.  In bfloat16 a token whose k-th and (k+1)-th choice scores lie within a rounding of each other is routed
# otherwise than the exact model routes it, and no bar on the logits survives that.  The bfloat16 models therefore have
# a quiet router and loud corrections: the corrections decide the choice, the router still sets the weights.  The
# float32 models route by their inputs; the choice itself is compared exactly in the kernel's own test.
STD_BY_NAME_QUIET = (("correction", 1.0), ("mlp.router", 0.002)) + STD_BY_NAME


def make_folder(tmp, name, store="float32"):
    from mashbox_b200.weights.random_init import write_model_folder
    cfg, seed, _ = CONFIGS[name]
    d = os.path.join(str(tmp), f"suf_{name}_{store}")
    if not os.path.isdir(d):
        write_model_folder(d, cfg, seed, dtype=getattr(torch, store), std=cfg.width ** -0.5, norm_std=0.1,
                           std_by_name=STD_BY_NAME if store == "float32" else STD_BY_NAME_QUIET)
    return d


@functools.lru_cache(maxsize=None)
def _model(folder):
    return read_model(folder)


@functools.lru_cache(maxsize=64)
def _logits(folder, tokens):
    cfg, W = _model(folder)
    return plain.forward(cfg, W, list(tokens)).numpy()


def plain_logits(folder, tokens):
    """float64 logits (T, V) of the plain implementation for one whole sequence"""
    return _logits(folder, tuple(int(t) for t in tokens))


def prompts_for(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0].vocab, n).tolist() for n in lengths]


def row_nmse(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return ((got - want) ** 2).sum(-1) / np.maximum((want ** 2).sum(-1), 1e-300)


# float32 against the float64 plain model: every product and sum is float32, measured 1e-13 to 1e-11 at these sizes.
# bfloat16 against the exact model: every sublayer's output is normed before it joins the stream, which brings a
# small output's rounding noise up to the stream's size; measured row by row 1e-4 to 8e-3 on these configurations
# (the mean over a prompt's rows 2e-4 to 1e-3), where a fault of a mechanism (a lost state, a latent too many, another
# expert) moves the rows by tens of percents.  So a row may reach 1e-2, a twentieth of the rows 1e-1, and the mean over
# the rows a fifth of the bar.  bfloat16 under another cut of the same tokens: the products run on other kernels with
# other orders of summation, so some values round to the neighbouring bfloat16; measured up to 6e-3 in a row, the mean
# below 5e-4.
BAR = {"float32": 1e-9, "bfloat16": 1e-2}
BAR_SAME = {"float32": 1e-11, "bfloat16": 1e-2}


def assert_close(got, want, dtype, what, bar=None):
    got = np.asarray(got, np.float64)
    assert got.shape == np.asarray(want).shape, (what, got.shape, np.asarray(want).shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = row_nmse(got, want)
    limit = (bar or BAR)[dtype]
    if dtype == "float32":
        assert e.max() <= limit, f"{what}: float32 NMSE {e.max():.3e} at row {int(e.argmax())}"
    else:
        over = int((e > limit).sum())
        mean = float(e.mean()) if len(e) >= 20 else 0.0
        assert over <= len(e) // 20 and e.max() <= 10 * limit and mean <= (limit / 5 if bar is None else limit / 10), \
            f"{what}: bfloat16: {over} of {len(e)} rows over {limit:.0e}, worst {e.max():.3e} at row {int(e.argmax())}, " \
            f"mean {e.mean():.3e}"
    return float(e.max())
