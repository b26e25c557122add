"""Plain, slow implementation of the Luzosun decoder: whole sequences, no cache, no state, one function per mechanism.

It is the oracle the engine is compared with and shares no code with ``mashbox_b200``: it reads config.json's keys
itself and works on CPU tensors in float64.  Angles of the rotation are formed in float32 first (as a 32-bit engine
forms them) and then widened.

The design, in this file's notation.  T tokens at positions 0 .. T-1, width D.

  x_0 = E[token] * s_e
  layer:   a = rms(x, w_1);  a' = a + causal_conv(a, c);  b = rms(x, w_2);  x <- x + (mixer(a') + ff(b))
  mixer:   q, k, v = causal_conv(W a' + bias) per projection; q and k hold two maps per head, [map 0 | map 1];
           the first R dims of every map are rotated (halves pairing) by position * theta^(-2i/R) / factor;
           s_m = softmax(scale * q_m k_m^T) under the mask "same block of M positions and not later";
           o = s_0 v - lam * s_1 v with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + delta;
           o <- o / sqrt(mean(o^2) + eps) * (1 - delta) per head; out = W_o concat(o)
           a layer may take k and v (as rotated and convolved by their owner) from an earlier layer
  ff:      W_down act(W_up b), act(z) = softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (e^z - 1 - z) + z/2 else
  logits = W_head rms(x, w_final)
"""
import math

import numpy as np
import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def causal_conv(u, w):
    """u (T, C), w (C, taps): y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start"""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def rotary_frequencies(base, dims, factor=None):
    """float32 angle per position step of pair i: base^(-2i/dims), divided by the linear factor"""
    i = np.arange(dims // 2, dtype=np.float32)
    f = (np.float32(base) ** (-2.0 * i / np.float32(dims))).astype(np.float32)
    if factor:
        f = (f / np.float32(factor)).astype(np.float32)
    return f


def rotate_halves(x, positions, freqs):
    """x (T, heads, dim): dims i and i + R/2 of the first R = 2 len(freqs) are one pair; the rest pass"""
    half = len(freqs)
    ang = (np.asarray(positions, np.float32)[:, None] * freqs[None, :]).astype(np.float32)
    c = torch.from_numpy(np.cos(ang.astype(np.float64)))[:, None, :]
    s = torch.from_numpy(np.sin(ang.astype(np.float64)))[:, None, :]
    a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([a * c - b * s, b * c + a * s, rest], -1)


def block_mask(T, size, start=0):
    """(T, T) bool: query i sees key j when j <= i and both lie in the same block of `size` positions (size None or
    0: every earlier key); positions are start + index"""
    p = torch.arange(start, start + T)
    m = p[None, :] <= p[:, None]
    if size:
        m = m & ((p[None, :] // size) == (p[:, None] // size))
    return m


def softmax_attention(q, k, v, scale, mask):
    """q (T, d), k (T, d), v (T, e) -> (T, e)"""
    s = (q @ k.T) * scale
    s = s.masked_fill(~mask, -math.inf)
    return torch.softmax(s, -1) @ v


def differential_lambda(lq1, lk1, lq2, lk2, delta):
    return math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + delta


def differential_heads(q, k, v, scale, mask, lam, delta, eps):
    """q (T, H, 2, d), k (T, G, 2, d), v (T, G, e) -> (T, H, e): the two maps of a head share the head's values"""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        a0 = softmax_attention(q[:, h, 0], k[:, g, 0], v[:, g], scale, mask)
        a1 = softmax_attention(q[:, h, 1], k[:, g, 1], v[:, g], scale, mask)
        out.append(rms(a0 - lam * a1, eps) * (1.0 - delta))
    return torch.stack(out, 1)


def xielu(z, p, q):
    sp = lambda t: math.log1p(math.exp(t))
    pos = sp(float(p)) * z * z + z / 2
    neg = (0.5 + sp(float(q))) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def feed_forward(b, W, p):
    act = W[p + "mlp.act"]
    return xielu(b @ W[p + "mlp.up"].T, act[0], act[1]) @ W[p + "mlp.down"].T


def projections(a, W, p, names, taps):
    """W a + bias, then (when the mixer has filters: `taps` given) the causal convolution of every channel"""
    out = {}
    for n in names:
        u = a @ W[p + "mix." + n].T + W[p + "mix." + n + ".b"]
        out[n] = causal_conv(u, W[p + "mix." + n + ".conv"]) if taps else u
    return out


def attention_mixer(a, W, p, m, eps, positions, shared):
    """a (T, D) -> (T, D); m: the layer's 'mixer' entry of config.json; shared: {layer: (k, v)} as their owners left
    them.  -> (output, (k, v) of this layer or None when it borrows them)"""
    T = a.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    freqs = None
    if rot:
        freqs = rotary_frequencies(rot["base"], rot["dims"], (rot.get("scaling") or {}).get("factor"))
    own = m.get("kv_from") is None
    pr = projections(a, W, p, ("q", "k", "v") if own else ("q",), m.get("conv"))
    q = pr["q"].reshape(T, H * 2, d)
    if freqs is not None:
        q = rotate_halves(q, positions, freqs)
    if own:
        k = pr["k"].reshape(T, G * 2, d)
        if freqs is not None:
            k = rotate_halves(k, positions, freqs)
        k, v = k.reshape(T, G, 2, d), pr["v"].reshape(T, G, e)
    else:
        k, v = shared[m["kv_from"]]
    mask = block_mask(T, (m.get("mask") or {}).get("size"), positions[0])
    lam = differential_lambda(W[p + "mix.lq1"], W[p + "mix.lk1"], W[p + "mix.lq2"], W[p + "mix.lk2"], m["diff"])
    o = differential_heads(q.reshape(T, H, 2, d), k, v, m["scale"], mask, lam, m["diff"], eps)
    return o.reshape(T, H * e) @ W[p + "mix.o"].T, ((k, v) if own else None)


def forward(cfg, W, tokens, layers_out=None):
    """-> float64 logits (T, vocab) of one whole sequence; layers_out: a list that receives the stream after each
    layer"""
    W = {k: v.to(F64) for k, v in W.items()}
    T = len(tokens)
    positions = np.arange(T)
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = rms(x, eps, W[p + "norm1"])
        if (cfg.get("canon") or {}).get("taps"):
            a = a + causal_conv(a, W[p + "canon1"])
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        y, kv = attention_mixer(a, W, p, layer["mixer"], eps, positions, shared)
        if kv is not None:
            shared[i] = kv
        if layer.get("mlp"):
            y = y + feed_forward(rms(x, eps, W[p + "norm2"]), W, p)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms(x, eps, W["final.norm"]) @ W["head"].T
