"""Small Luzosun configurations with random weights, and the plain implementation's logits for them."""
import functools
import os

import numpy as np
import torch

from mashbox_b200.config.luzosun import LuzosunConfig, LuzosunLayer, LuzosunMixer
from tests.plain import luzosun as plain
from tests.plain.llama import read_model


def mixer(heads, kv, dim, vdim, diff, conv, mask, rot, kv_from=None, scale=None):
    base, dims, factor = rot if rot else (None, 0, None)
    return LuzosunMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, diff=diff, scale=scale or dim ** -0.5, conv=conv,
                        mask_size=mask, rot_base=base, rot_dims=dims, rot_factor=factor, kv_from=kv_from)


# P: every size differs from layer to layer where it may; blocks of 20 positions (no multiple of the page size) and
#    of 48; three query heads per kv head and one; a layer that borrows keys and values and has no feed-forward.
_p0 = mixer(6, 2, 16, 40, 0.25, 3, 20, (10000.0, 8, 2.0))
_p2 = mixer(2, 2, 24, 24, 0.4, 5, 48, (500.0, 24, None), scale=0.3)
LUZ_P = LuzosunConfig("Luzosun", width=64, vocab=211, embedding_scale=4.0, norm_eps=1e-5, canon_taps=2, layers=(
    LuzosunLayer("attention", _p0, 96),
    LuzosunLayer("attention", mixer(6, 2, 16, 40, 0.1, 2, 40, (10000.0, 8, 2.0), kv_from=0), None),
    LuzosunLayer("attention", _p2, 160),
    LuzosunLayer("attention", mixer(2, 2, 24, 24, 0.4, 5, 48, (500.0, 24, None), kv_from=2, scale=0.2), 72)))
# Q: what P does not have: no mask (every earlier key), no rotation, no q/k/v convolutions in one layer and filters of ONE
#    tap in another (they keep no state), no input convolution, one kv head, embedding scale 1
LUZ_Q = LuzosunConfig("Luzosun", width=96, vocab=130, embedding_scale=1.0, norm_eps=1e-6, canon_taps=0, layers=(
    LuzosunLayer("attention", mixer(4, 1, 32, 32, 0.5, None, None, None), 128),
    LuzosunLayer("attention", mixer(4, 4, 16, 48, 0.2, 4, 32, (30000.0, 16, 2.0)), 64),
    LuzosunLayer("attention", mixer(2, 2, 16, 32, 0.0, 1, 1, (100.0, 16, None)), 40)))
# R: head sizes the tensor-core attention kernel takes (multiples of 16), blocks of 64 and 128 positions
# S: an input convolution of ONE tap (no state at all in a layer whose mixer has no filters), a mask of 3 positions
LUZ_S = LuzosunConfig("Luzosun", width=40, vocab=97, embedding_scale=2.5, norm_eps=1e-5, canon_taps=1, layers=(
    LuzosunLayer("attention", mixer(2, 1, 8, 24, 0.45, None, 3, (10000.0, 4, None)), 48),
    LuzosunLayer("attention", mixer(2, 1, 8, 24, 0.6, 2, 7, (10000.0, 4, None), kv_from=0), None)))
LUZ_R = LuzosunConfig("Luzosun", width=128, vocab=301, embedding_scale=8.0, norm_eps=2e-6, canon_taps=3, layers=(
    LuzosunLayer("attention", mixer(4, 2, 32, 64, 0.35, 5, 64, (50000.0, 16, 8.0)), 192),
    LuzosunLayer("attention", mixer(4, 2, 32, 64, 0.25, 2, 128, (50000.0, 16, 8.0), kv_from=0), 192),
    LuzosunLayer("attention", mixer(2, 1, 64, 128, 0.2, 3, 64, (1000.0, 64, None)), 96)))
CONFIGS = {"P": (LUZ_P, 5, 8), "Q": (LUZ_Q, 6, 16), "R": (LUZ_R, 7, 16), "S": (LUZ_S, 8, 4)}       # config, seed, page size

# Readers near 1/sqrt(fan in), writers into the stream small, filters and the vectors of lambda of order 0.3: the
# stream stays of order one and attention is not uniform.
STD_BY_NAME = ((".conv", 0.3), ("canon1", 0.3), (".b", 0.1), ("mix.l", 0.3), ("mlp.act", 0.7), ("mix.o", 0.03),
               ("mlp.down", 0.03), ("embed", 0.5))


def make_folder(tmp, name, store="float32"):
    from mashbox_b200.weights.random_init import write_model_folder
    cfg, seed, _ = CONFIGS[name]
    d = os.path.join(str(tmp), f"luz_{name}_{store}")
    if not os.path.isdir(d):
        write_model_folder(d, cfg, seed, dtype=getattr(torch, store), std=cfg.width ** -0.5, norm_std=0.1,
                           std_by_name=STD_BY_NAME)
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


def nmse(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(((got - want) ** 2).sum() / max((want ** 2).sum(), 1e-300))


# float32: every product and sum is float32, NMSE around 1e-12 at these sizes.  bfloat16 against the exact model: a
# dozen roundings of 2^-9 per layer, measured 2e-5 to 6e-5 on these configurations; a fault of the mechanisms (a key
# too many, a lost state) moves the logits by percents.  bfloat16 against bfloat16 under another cut of the same
# tokens: the same roundings at the same places, what differs is the order of float32 sums before a rounding.
BAR = {"float32": 1e-10, "bfloat16": 4e-4}
BAR_SAME = {"float32": 1e-11, "bfloat16": 3e-5}


def assert_close(got, want, dtype, what, bar=None):
    got = np.asarray(got, np.float64)
    assert got.shape == np.asarray(want).shape, (what, got.shape, np.asarray(want).shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = nmse(got, want)
    assert e <= (bar or BAR)[dtype], f"{what}: {dtype} NMSE {e:.3e}"
    return e
