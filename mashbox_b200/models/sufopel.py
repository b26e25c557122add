"""The Sufopel decoder as data: which parts each layer has, in which order layers run, whose latents each reads and
which tensors exist under which names.

Token rows plus a learned position vector enter the stream.  Every layer is a sandwich block -- a norm before and
after each sublayer, the normed output scaled per channel -- whose mixer is either latent attention (one latent vector
kept per position; a layer may read the latents of an earlier layer) or the channel-wise gated delta rule (a matrix
state per head and request, nothing kept per position), whose feed-forward is dense SwiGLU, routed experts or absent,
and which ends with an input from the token itself when the model has a second embedding table.  A layer that reads
another layer's latents names that layer's cache read-only in its schedule entry; a delta layer names no cache and a
state of its own.  Stored names: `embed`, `pos`, `side.embed`, `l<i>.norm1|norm1b|norm2|norm2b|ls1|ls2`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down` or `l<i>.mlp.router|correction|e<j>.gate|up|down`, `l<i>.side.gate|proj|norm`, `final.norm`,
`head`.
"""
from ..config.sufopel import DenseFF, SufopelConfig
from ..parts.base import LayerRun, LayerSpec, ModelSpec, PartSpec

DEFAULT_RANK = 16       # inner width of a delta layer's low-rank products when random weights are made and none is given


def model_spec(c: SufopelConfig) -> ModelSpec:
    D = c.width
    norm = PartSpec("rms", width=D, eps=c.norm_eps)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", hidden=D, heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank,
                             kv_rank=m.kv_rank, eps=c.norm_eps, scale=m.scale, gate=True, shares_kv=m.kv_from is not None,
                             names={k: "mix." + v for k, v in dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv",
                                                                   dkv_norm="dkv.norm", uk="uk", uv="uv", g="g", o="o").items()})
            own = m.kv_from is None
            run = LayerRun(layer=i, cache=i if own else m.kv_from, write=own)
        else:
            mixer = PartSpec("channel_delta", hidden=D, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                             eps=c.norm_eps, taps=m.conv, decay_rank=m.a_rank, gate_rank=m.g_rank,
                             names={k: "mix." + v for k, v in dict(q="q", k="k", v="v", b="b", A="A_log", norm="norm", a1="a1",
                                                                   a2="a2", dt="dt_bias", g1="g1", g2="g2", o="o").items()})
            run = LayerRun(layer=i, cache=None, write=False, state=i)
        f = layer.mlp
        if f is None:
            ffn = None
        elif isinstance(f, DenseFF):
            ffn = PartSpec("swiglu", hidden=D, intermediate=f.ff, names=dict(gate="mlp.gate", up="mlp.up", down="mlp.down"))
        else:
            ffn = PartSpec("routed_experts", hidden=D, intermediate=f.ff, experts=f.experts, top=f.top, limit=f.limit,
                           groups=f.groups, keep=f.keep)
        side = None
        if c.side_dim:
            side = PartSpec("gated_table", hidden=D, dim=c.side_dim, offset=i * c.side_dim,
                            table_width=c.num_layers * c.side_dim, vocab=c.vocab, eps=c.norm_eps)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("sandwich", mixer=mixer, ffn=ffn, norm=norm, side=side,
                                                                 scale1="ls1", scale2="ls2")))
        schedule.append(run)
    return ModelSpec(hidden=D, vocab=c.vocab,
                     embedding=PartSpec("table_positions", vocab=c.vocab, hidden=D, max_positions=c.max_positions,
                                        name="embed", position_name="pos", scale=c.embedding_scale),
                     layers=layers, schedule=schedule,
                     final_norm=PartSpec("rms", width=D, eps=c.norm_eps, name="final.norm"),
                     head=PartSpec("linear", vocab=c.vocab, hidden=D, tied=False, name="head", scale=c.logit_scale))


def canonical_names(c: SufopelConfig):
    """stored names are the canonical ones, except that the dense feed-forward's matrices get the `.weight` its part
    appends; a name outside the configuration's table is unexpected"""
    known = set(stored_tensors(c))
    dense = {f"l{i}.mlp.{r}" for i, layer in enumerate(c.layers) if isinstance(layer.mlp, DenseFF) for r in ("gate", "up", "down")}

    def canonical(name):
        if name not in known:
            raise KeyError(name)
        return (name + ".weight" if name in dense else name), None
    return canonical


def stored_tensors(c: SufopelConfig):
    """names, shapes and kinds of the tensors a checkpoint of this configuration holds"""
    D = c.width
    out = {"embed": ((c.vocab, D), "matrix"), "pos": ((c.max_positions, D), "matrix")}
    if c.side_dim:
        out["side.embed"] = ((c.vocab, c.num_layers * c.side_dim), "matrix")
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer.mixer
        for n in ("norm1", "norm1b"):
            out[p + n] = ((D,), "norm")
        out[p + "ls1"] = ((D,), "bias")
        x = p + "mix."
        if layer.type == "latent_attention":
            out[x + "dq"] = ((m.q_rank, D), "matrix")
            out[x + "dq.norm"] = ((m.q_rank,), "norm")
            out[x + "uq"] = ((m.heads * m.dim, m.q_rank), "matrix")
            if m.kv_from is None:
                out[x + "dkv"] = ((m.kv_rank, D), "matrix")
                out[x + "dkv.norm"] = ((m.kv_rank,), "norm")
            out[x + "uk"] = ((m.heads * m.dim, m.kv_rank), "matrix")
            out[x + "uv"] = ((m.heads * m.vdim, m.kv_rank), "matrix")
            out[x + "g"] = ((m.heads * m.vdim, D), "matrix")
            out[x + "o"] = ((D, m.heads * m.vdim), "matrix")
        else:
            ra, rg = m.a_rank or DEFAULT_RANK, m.g_rank or DEFAULT_RANK
            for r, rows in (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim)):
                out[x + r] = ((rows, D), "matrix")
                if m.conv:
                    out[x + r + ".conv"] = ((rows, m.conv), "matrix")
            out[x + "b"] = ((m.heads, D), "matrix")
            out[x + "A_log"] = ((m.heads,), "bias")
            out[x + "norm"] = ((m.vdim,), "norm")
            out[x + "a1"] = ((ra, D), "matrix")
            out[x + "a2"] = ((m.heads * m.dim, ra), "matrix")
            out[x + "dt_bias"] = ((m.heads * m.dim,), "bias")
            out[x + "g1"] = ((rg, D), "matrix")
            out[x + "g2"] = ((m.heads * m.vdim, rg), "matrix")
            out[x + "o"] = ((D, m.heads * m.vdim), "matrix")
        f = layer.mlp
        if f is not None:
            for n in ("norm2", "norm2b"):
                out[p + n] = ((D,), "norm")
            out[p + "ls2"] = ((D,), "bias")
            if isinstance(f, DenseFF):
                out[p + "mlp.gate"] = ((f.ff, D), "matrix")
                out[p + "mlp.up"] = ((f.ff, D), "matrix")
                out[p + "mlp.down"] = ((D, f.ff), "matrix")
            else:
                for e in range(f.experts):
                    out[f"{p}mlp.e{e}.gate"] = ((f.ff, D), "matrix")
                    out[f"{p}mlp.e{e}.up"] = ((f.ff, D), "matrix")
                    out[f"{p}mlp.e{e}.down"] = ((D, f.ff), "matrix")
                out[p + "mlp.router"] = ((f.experts, D), "matrix")
                out[p + "mlp.correction"] = ((f.experts,), "bias")
        if c.side_dim:
            out[p + "side.gate"] = ((c.side_dim, D), "matrix")
            out[p + "side.proj"] = ((D, c.side_dim), "matrix")
            out[p + "side.norm"] = ((D,), "norm")
    out["final.norm"] = ((D,), "norm")
    out["head"] = ((c.vocab, D), "matrix")
    return out
