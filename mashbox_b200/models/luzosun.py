"""The Luzosun decoder as data: which parts each layer has, in which order layers run and whose cache each reads,
which tensors exist under which names.

Every layer is a parallel block -- the mixer and the feed-forward read the same stream through norms of their own --
with a short convolution on what the mixer reads, a differential attention mixer (two softmax maps per head, short
convolutions on q/k/v, partial rotation with linearly scaled frequencies, a mask of blocks of positions) and a dense
feed-forward with the xIELU activation.  A layer may read the keys and values of an earlier layer: its schedule entry
names that layer's cache, read-only, and a state of its own.  Stored names are the canonical names: `embed`,
`l<i>.norm1|norm2|canon1`, `l<i>.mix.q|k|v` (+ `.b`, `.conv`), `l<i>.mix.lq1|lk1|lq2|lk2|o`, `l<i>.mlp.up|down|act`,
`final.norm`, `head`.
"""
from ..config.luzosun import LuzosunConfig
from ..parts.base import LayerRun, LayerSpec, ModelSpec, PartSpec


def model_spec(c: LuzosunConfig) -> ModelSpec:
    D = c.width
    norm = PartSpec("rms", width=D, eps=c.norm_eps)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        rope = None
        if m.rot_base is not None:
            rope = PartSpec("rope", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base, pairing="halves",
                            scaling=("divide", m.rot_factor) if m.rot_factor else None)
        mixer = PartSpec("differential_attention", hidden=D, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                         delta=m.diff, eps=c.norm_eps, scale=m.scale, bias=True, taps=m.conv, position=rope,
                         chunk=m.mask_size, shares_kv=m.kv_from is not None,
                         names=dict(q="mix.q", k="mix.k", v="mix.v", o="mix.o", lq1="mix.lq1", lk1="mix.lk1",
                                    lq2="mix.lq2", lk2="mix.lk2"))
        ffn = None
        if layer.ff:
            ffn = PartSpec("dense_xielu", hidden=D, intermediate=layer.ff,
                           names=dict(up="mlp.up", down="mlp.down", act="mlp.act"))
        conv = PartSpec("short", channels=D, taps=c.canon_taps, residual=True) if c.canon_taps >= 1 else None
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("parallel", mixer=mixer, ffn=ffn, norm1=norm,
                                                                 mixer_conv=conv)))
        own = m.kv_from is None
        schedule.append(LayerRun(layer=i, cache=i if own else m.kv_from, write=own, state=i))
    return ModelSpec(hidden=D, vocab=c.vocab,
                     embedding=PartSpec("table", vocab=c.vocab, hidden=D, name="embed", scale=c.embedding_scale),
                     layers=layers, schedule=schedule,
                     final_norm=PartSpec("rms", width=D, eps=c.norm_eps, name="final.norm"),
                     head=PartSpec("linear", vocab=c.vocab, hidden=D, tied=False, name="head"))


def canonical_names(c: LuzosunConfig):
    """stored names are the canonical ones; a name outside the configuration's table is unexpected"""
    known = set(stored_tensors(c))

    def canonical(name):
        if name not in known:
            raise KeyError(name)
        return name, None
    return canonical


def stored_tensors(c: LuzosunConfig):
    """names, shapes and kinds of the tensors a checkpoint of this configuration holds"""
    D = c.width
    out = {"embed": ((c.vocab, D), "matrix")}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        out[p + "norm1"] = ((D,), "norm")
        rows = {"q": m.heads * 2 * m.dim}
        if m.kv_from is None:
            rows.update(k=m.kv_heads * 2 * m.dim, v=m.kv_heads * m.vdim)
        for r, n in rows.items():
            out[p + "mix." + r] = ((n, D), "matrix")
            out[p + "mix." + r + ".b"] = ((n,), "bias")
            if m.conv:
                out[p + "mix." + r + ".conv"] = ((n, m.conv), "matrix")
        for v in ("lq1", "lk1", "lq2", "lk2"):
            out[p + "mix." + v] = ((m.dim,), "bias")
        out[p + "mix.o"] = ((D, m.heads * m.vdim), "matrix")
        if layer.ff:
            out[p + "norm2"] = ((D,), "norm")
            out[p + "mlp.up"] = ((layer.ff, D), "matrix")
            out[p + "mlp.down"] = ((D, layer.ff), "matrix")
            out[p + "mlp.act"] = ((2,), "bias")
        if c.canon_taps >= 1:
            out[p + "canon1"] = ((D, c.canon_taps), "matrix")
    out["final.norm"] = ((D,), "norm")
    out["head"] = ((c.vocab, D), "matrix")
    return out
