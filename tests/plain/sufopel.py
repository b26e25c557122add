"""Plain, slow implementation of the Sufopel decoder: whole sequences, no cache, no state carried between calls, one
function per mechanism.

It is the oracle the engine is compared with and shares no code with ``mashbox_b200``: it reads config.json's keys
itself (a dict) and works on CPU tensors in float64.

The design, in this file's notation.  T tokens at positions 0 .. T-1, width D, rms(x) = x / sqrt(mean(x^2) + eps).

  x_0     = E[token] * s_e + P[position]
  layer i : x <- x + l1 * (rms(mixer(rms(x) w1)) w1b);  x <- x + l2 * (rms(ff(rms(x) w2)) w2b)
            then the token's own input:  e = Es[token, i d : (i+1) d];  y = Wp (gelu_tanh(Wg x) * e);
            x <- x + rms(y) ws
  latent attention:  cq = rms(Wdq h) nq;  q = Wuq cq;  c = rms(Wdkv h) nkv (or another layer's c);  k = Wuk c;
            v = Wuv c;  causal softmax(scale q k^T) v per head;  times sigmoid(Wg h);  Wo
  channel delta:  q, k, v = silu(causal_conv(W h));  q, k unit vectors per head (q also times dim^-1/2);
            beta = sigmoid(Wb h);  g = exp(-exp(A) softplus(Wa2 Wa1 h + dt)) per head and key channel;
            per token  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
            o <- rms(o) n * sigmoid(Wg2 Wg1 h);  Wo
  ff dense: Wd (silu(Wg h) * (Wu h))
  ff routed: s = sigmoid(Wr h); c = s + correction; experts outside the best groups (a group's score: its two largest
            c) get c = -inf; the `top` largest c are chosen; out = sum of s_e expert_e(h) over the chosen;
            expert: g = min(Wg h, L); u = clamp(Wu h, -L, L); Wd (g sigmoid(1.702 g) (u + 1))
  logits  = W_head (rms(x) w_final) * s_l
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, w):
    """u (T, C), w (C, taps): y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start"""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def embed(W, cfg, tokens):
    t = torch.as_tensor(tokens, dtype=torch.long)
    return W["embed"][t] * float(cfg["embedding"]["scale"]) + W["pos"][torch.arange(len(t))]


def latent_of(W, p, h, eps):
    """the latent a layer keeps per position"""
    return rms(h @ W[p + "mix.dkv"].T, eps, W[p + "mix.dkv.norm"])


def latent_attention(W, p, m, h, c, eps):
    """h (T, D) the mixer's input, c (T, kv_rank) the latents it attends to (its own or another layer's)"""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    cq = rms(h @ W[p + "mix.dq"].T, eps, W[p + "mix.dq.norm"])
    q = (cq @ W[p + "mix.uq"].T).view(T, H, dim)
    k = (c @ W[p + "mix.uk"].T).view(T, H, dim)
    v = (c @ W[p + "mix.uv"].T).view(T, H, vdim)
    score = torch.einsum("thd,shd->hts", q, k) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    score = score.masked_fill(~mask, -math.inf)
    a = torch.softmax(score, -1)
    o = torch.einsum("hts,shd->thd", a, v).reshape(T, H * vdim)
    o = o * torch.sigmoid(h @ W[p + "mix.g"].T)
    return o @ W[p + "mix.o"].T


def delta_rule(q, k, v, g, beta):
    """q, k, g (T, dim), v (T, vdim), beta (T,) of one head -> o (T, vdim); the state starts at zero"""
    T, dim = q.shape
    S = torch.zeros(dim, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def channel_delta(W, p, m, h, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def branch(name):
        z = h @ W[p + "mix." + name].T
        if m.get("conv"):
            z = causal_conv(z, W[p + "mix." + name + ".conv"])
        return silu(z)
    q = branch("q").view(T, G, dim)
    k = branch("k").view(T, G, dim)
    v = branch("v").view(T, H, vdim)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * dim ** -0.5, unit(k)
    beta = torch.sigmoid(h @ W[p + "mix.b"].T)                                  # (T, H)
    dt = (h @ W[p + "mix.a1"].T) @ W[p + "mix.a2"].T + W[p + "mix.dt_bias"]
    g = torch.exp(-torch.exp(W[p + "mix.A_log"])[None, :, None] * torch.nn.functional.softplus(dt).view(T, H, dim))
    gate = torch.sigmoid((h @ W[p + "mix.g1"].T) @ W[p + "mix.g2"].T).view(T, H, vdim)
    outs = []
    for hd in range(H):
        j = hd // (H // G)
        o = delta_rule(q[:, j], k[:, j], v[:, hd], g[:, hd], beta[:, hd])
        outs.append(rms(o, eps, W[p + "mix.norm"]) * gate[:, hd])
    return torch.cat(outs, -1) @ W[p + "mix.o"].T


def dense_ff(W, p, h):
    return (silu(h @ W[p + "mlp.gate"].T) * (h @ W[p + "mlp.up"].T)) @ W[p + "mlp.down"].T


def route(W, p, r, h):
    """-> (chosen experts (T, top), their weights (T, top))"""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ W[p + "mlp.router"].T)
    c = s + W[p + "mlp.correction"]
    groups = r.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = c.view(-1, n, E // n)
        score = per.topk(min(2, E // n), -1).values.sum(-1)                     # (T, n)
        best = score.topk(keep, -1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        c = per.masked_fill(~allowed[:, :, None], -math.inf).reshape(-1, E)
    chosen = c.topk(top, -1).indices
    return chosen, s.gather(1, chosen)


def expert(W, p, e, h, limit):
    g = torch.clamp(h @ W[f"{p}mlp.e{e}.gate"].T, max=limit)
    u = torch.clamp(h @ W[f"{p}mlp.e{e}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[f"{p}mlp.e{e}.down"].T


def routed_ff(W, p, mlp, h):
    chosen, weight = route(W, p, mlp["router"], h)
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros(h.shape[0], W[p + "mlp.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weight[t]):
            out[t] = out[t] + w * expert(W, p, e, h[t:t + 1], limit)[0]
    return out


def token_side(W, p, i, dim, x, tokens, eps):
    e = W["side.embed"][torch.as_tensor(tokens, dtype=torch.long)][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
    return rms(y, eps, W[p + "side.norm"])


def forward(cfg, W, tokens, layers_out=None):
    """cfg: config.json as a dict; W: {name: float64 tensor}; tokens: ids -> logits (T, vocab) float64.
    layers_out: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(W, cfg, tokens)
    latents = {}
    side = (cfg.get("token_side") or {}).get("dim")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms(x, eps, W[p + "norm1"])
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(W, p, h, eps)
            y = latent_attention(W, p, m, h, latents[i if src is None else src], eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(W, p, m, h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms(y, eps, W[p + "norm1b"]) * W[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms(x, eps, W[p + "norm2"])
            y = dense_ff(W, p, h) if mlp.get("kind", "dense") == "dense" else routed_ff(W, p, mlp, h)
            x = x + rms(y, eps, W[p + "norm2b"]) * W[p + "ls2"]
        if side:
            x = x + token_side(W, p, i, int(side), x, tokens, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps, W["final.norm"]) @ W["head"].T) * float(cfg.get("logit_scale", 1.0))
