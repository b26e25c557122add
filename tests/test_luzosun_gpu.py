"""-m gpu: the Luzosun decoder in the engine against the plain implementation (tests/plain/luzosun.py), in float32 and
bfloat16: single kernels on inputs built so that a fault shows (one loud key just inside or just outside a block of
positions, far back, at a page's border), whole prompts, prefill against token-by-token decoding, portions down to one
and two tokens, batches of unequal requests against each alone, pages and state slots used again, long decoding over
several blocks, and greedy generation through the engine's own entry point and scheduler."""
import numpy as np
import pytest
import torch

from tests import luzosun_helpers as L
from tests.gpu_harness import DEV, i32
from tests.plain import luzosun as plain

pytestmark = pytest.mark.gpu
DTYPES = ("float32", "bfloat16")
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_BAR = {"float32": 2e-5, "bfloat16": 2e-2}          # of the largest value


def kernel_close(got, want, dtype, what):
    got, want = np.asarray(got.detach().float().cpu(), np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert np.isfinite(got).all() and err <= KERNEL_BAR[dtype], f"{what}: {dtype} worst error {err:.3e} of the largest value"


# ------------------------------------------------------------------------------------------------ single kernels
def seq_arrays(q_lens, slots):
    q_start = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
    tok_seq = np.repeat(np.arange(len(q_lens)), q_lens)
    return (i32(tok_seq), i32(q_start), i32(q_lens), i32(slots))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C", [40, 37])          # eight channels a thread, and the widths that form does not take
@pytest.mark.parametrize("taps,residual", [(2, True), (4, False), (5, True), (8, False), (1, True)])
def test_short_conv_carries_its_state_across_any_cut(dtype, taps, residual, C):
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(taps)
    T = 37
    u = [torch.randn(T, C, generator=g).to(TD[dtype]).double() for _ in range(3)]
    w = torch.randn(C, taps, generator=g)
    want = [plain.causal_conv(x, w.double()) + (x if residual else 0) for x in u]
    pad = 24                                                             # the stretch lies inside a wider state tensor
    state = torch.zeros(5, pad + (taps - 1) * C + 8, device=DEV)
    view = state[:, pad:pad + (taps - 1) * C] if taps > 1 else None
    slots = [3, 0, 4]
    # the three sequences advance by portions of their own sizes, 1 and 2 tokens among them, side by side
    cuts = [[1, 1, 1, 2, 5, 1, 9, 3, 14], [2, 2, 1, 7, 25], [taps - 1 or 1, taps, taps + 1, 1, 2]]
    cuts[2].append(T - sum(cuts[2]))
    at = [0, 0, 0]
    got = [[], [], []]
    step = 0
    while any(a < T for a in at):
        live = [s for s in range(3) if at[s] < T and step < len(cuts[s])]
        lens = [cuts[s][step] for s in live]
        x = torch.cat([u[s][at[s]:at[s] + n] for s, n in zip(live, lens)]).to(DEV, TD[dtype]).contiguous()
        out = torch.empty_like(x)
        ops.short_conv(x, w.t().contiguous().to(DEV), view, seq_arrays(lens, [slots[s] for s in live]), out, residual)
        o = 0
        for s, n in zip(live, lens):
            got[s].append(out[o:o + n])
            o += n
            at[s] += n
        step += 1
    for s in range(3):
        kernel_close(torch.cat(got[s]), want[s], dtype, f"short convolution of {taps} taps, sequence {s}")
    assert float(state[:, :pad].abs().max()) == 0 and float(state[:, pad + (taps - 1) * C:].abs().max()) == 0
    assert float(state[1].abs().max()) == 0 and float(state[2].abs().max()) == 0      # slots nobody has


@pytest.mark.parametrize("dtype", DTYPES)
def test_xielu_and_pair_of_norms(dtype):
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(3)
    for N, F in ((5, 24), (3, 37)):
        z = (3 * torch.randn(N, F, generator=g)).to(TD[dtype])
        out = torch.empty(N, F, device=DEV, dtype=TD[dtype])
        sp = lambda t: float(np.log1p(np.exp(t)))
        ops.xielu(z.to(DEV).contiguous(), out, sp(0.4), 0.5 + sp(-0.3))
        kernel_close(out, plain.xielu(z.double(), 0.4, -0.3), dtype, f"xIELU {N}x{F}")
    for D in (64, 52):
        x = torch.randn(6, D, generator=g)
        d1, d2 = (torch.randn(6, D, generator=g).to(TD[dtype]) for _ in range(2))
        w1, w2 = 1 + 0.1 * torch.randn(D, generator=g), 1 + 0.1 * torch.randn(D, generator=g)
        v = x.double() + d1.double() + d2.double()
        xs = x.to(DEV)
        a, b = (torch.empty(6, D, device=DEV, dtype=TD[dtype]) for _ in range(2))
        ops.add_rmsnorm_pair(xs, d1.to(DEV), d2.to(DEV), w1.to(DEV), w2.to(DEV), 1e-5, a, b)
        kernel_close(xs, v, "float32", "the stream after both adds")
        kernel_close(a, plain.rms(v, 1e-5, w1.double()), dtype, f"first norm, width {D}")
        kernel_close(b, plain.rms(v, 1e-5, w2.double()), dtype, f"second norm, width {D}")
        rows = i32([4, 1])
        xs2 = x.to(DEV)
        r = torch.empty(2, D, device=DEV, dtype=TD[dtype])
        ops.add_rmsnorm_pair(xs2, d1.to(DEV), None, w1.to(DEV), None, 1e-5, r, None, rows)
        kernel_close(r, plain.rms((x.double() + d1.double())[[4, 1]], 1e-5, w1.double()), dtype, "picked rows")
        assert torch.equal(xs2.cpu(), x)                                  # picked rows leave the stream alone


def test_up_product_with_the_activation_in_its_epilogue():
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(9)
    sp = lambda t: float(np.log1p(np.exp(t)))
    for N, K, F in ((200, 64, 96), (129, 72, 264)):
        if not ops.fused_xielu_supports(N, F, K):
            pytest.skip("the fused product does not take these sizes")
        x = torch.randn(N, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(F, K, generator=g) * K ** -0.5 * 2).to(torch.bfloat16)
        out = torch.empty(N, F, device=DEV, dtype=torch.bfloat16)
        ops.linear_xielu(x.to(DEV), w.to(DEV), out, sp(0.4), 0.5 + sp(-0.3))
        kernel_close(out, plain.xielu(x.double() @ w.double().T, 0.4, -0.3), "bfloat16", f"fused up product {N}x{K}x{F}")
    ops.check_error_word(ops.error_word(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_of_norms_with_the_convolution_folded_in_is_the_two_kernels(dtype):
    """one-token stretches: the norm kernel with the input convolution folded in leaves the same bits, in its outputs
    and in the state, as the norm kernel followed by the convolution kernel"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(5)
    N, D, taps = 5, 72, 4
    w1, w2 = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV), (1 + 0.1 * torch.randn(D, generator=g)).to(DEV)
    cw = torch.randn(taps, D, generator=g).to(DEV)
    slots = [4, 0, 2, 5, 1]
    states = [torch.zeros(7, 16 + (taps - 1) * D, device=DEV) for _ in range(2)]
    views = [s[:, 16:] for s in states]
    xs = [torch.randn(N, D, generator=g).to(DEV).clone() for _ in range(2)]
    xs[1].copy_(xs[0])
    for step in range(6):                                                 # the state fills up and then shifts
        d1, d2 = (torch.randn(N, D, generator=g).to(TD[dtype]).to(DEV) for _ in range(2))
        a0, b0, a1, b1, c0 = (torch.empty(N, D, device=DEV, dtype=TD[dtype]) for _ in range(5))
        ops.add_rmsnorm_pair(xs[0], d1, d2, w1, w2, 1e-5, a0, b0)
        ops.short_conv(a0, cw, views[0], seq_arrays([1] * N, slots), c0, True)
        ops.add_rmsnorm_pair_conv(xs[1], d1, d2, w1, w2, 1e-5, a1, b1, cw, views[1], i32(slots))
        assert torch.equal(c0, a1) and torch.equal(b0, b1) and torch.equal(xs[0], xs[1]), f"step {step}"
        assert torch.equal(states[0], states[1]), f"state after step {step}"


class DiffCase:
    """S sequences with two-map queries and keys in shuffled pages; the step's queries are each sequence's last ones"""

    def __init__(self, lengths, q_lens, H, G, dim, vdim, page, dtype, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.q_lens, self.H, self.G, self.dim, self.vdim, self.page = lengths, q_lens, H, G, dim, vdim, page
        self.dtype = dtype
        r = lambda *s: torch.randn(*s, generator=g).to(TD[dtype]).double()
        self.q = [r(n, H, 2, dim) for n in lengths]
        self.k = [r(n, G, 2, dim) for n in lengths]
        self.v = [r(n, G, vdim) for n in lengths]
        self.gen = g

    def build(self):
        page, G = self.page, self.G
        blocks = [-(-n // page) for n in self.lengths]
        pages = sum(blocks) + 3
        perm = torch.randperm(pages, generator=self.gen).tolist()
        self.table = np.full((len(self.lengths), max(blocks) + 1), -1, np.int32)
        fill = float("nan") if self.dtype == "float32" else 0.0          # a read past a sequence's end shows in float32
        kpool = torch.full((pages, G, page, 2 * self.dim), fill, dtype=torch.float64)
        vpool = torch.full((pages, G, page, self.vdim), fill, dtype=torch.float64)
        nxt = 0
        for s, n in enumerate(self.lengths):
            for b in range(blocks[s]):
                pg = perm[nxt]
                nxt += 1
                self.table[s, b] = pg
                lo, hi = b * page, min(n, (b + 1) * page)
                kpool[pg, :, :hi - lo] = self.k[s][lo:hi].reshape(hi - lo, G, -1).transpose(0, 1)
                vpool[pg, :, :hi - lo] = self.v[s][lo:hi].transpose(0, 1)
        self.pages = pages
        self.kpool, self.vpool = kpool.to(DEV, TD[self.dtype]).contiguous(), vpool.to(DEV, TD[self.dtype]).contiguous()
        self.positions = np.concatenate([np.arange(n - q, n) for n, q in zip(self.lengths, self.q_lens)])
        self.tok_row = np.repeat(np.arange(len(self.lengths)), self.q_lens)
        qs = torch.cat([self.q[s][n - q:] for s, (n, q) in enumerate(zip(self.lengths, self.q_lens))])
        self.N = qs.shape[0]
        self.q_dev = qs.reshape(self.N, -1).to(DEV, TD[self.dtype]).contiguous()
        return self

    def reference(self, scale, chunk, lam, delta, eps):
        out = []
        for s, (n, ql) in enumerate(zip(self.lengths, self.q_lens)):
            o = plain.differential_heads(self.q[s], self.k[s], self.v[s], scale, plain.block_mask(n, chunk), lam, delta, eps)
            out.append(o[n - ql:].reshape(ql, -1))
        return torch.cat(out)


def run_diff(case, chunk, scale, lam, delta, eps, kernel="simple"):
    """kernel: "simple", "mma" (the plan the mixer makes), "mma-N" (decode-form sequences cut into N splits) or "tc5"
    (prompt-form sequences on the tcgen05 kernel)"""
    from mashbox_b200 import ops
    from mashbox_b200.parts.diff_attention import plan_diff_attention
    out = torch.empty(case.N, case.H * case.vdim, device=DEV, dtype=TD[case.dtype])
    err = ops.new_error_word(DEV)
    args = (case.H, case.G, case.dim, case.vdim, case.page, case.pages, chunk, scale, lam, 1.0 - delta, eps, err)
    if kernel == "simple":
        ops.attention_diff_simple(case.q_dev, out, i32(case.positions), i32(case.tok_row), i32(case.table), case.kpool,
                                  case.vpool, *args)
    else:
        q_start = np.concatenate([[0], np.cumsum(case.q_lens)[:-1]])
        pos0 = [n - q for n, q in zip(case.lengths, case.q_lens)]
        tc5 = kernel == "tc5"
        plan = plan_diff_attention(case.q_lens, pos0, case.H // case.G, case.G, chunk,
                                   ops.attention_tc5_diff_rows() if tc5 else ops.attention_diff_mma_rows(),
                                   splits=int(kernel[4:]) if "-" in kernel else None, quads=tc5)
        seqs = (i32(q_start), i32(case.q_lens), i32(pos0), i32(np.arange(len(case.lengths))))
        tail = (i32(case.table), case.kpool, case.vpool) + args
        if plan["pre"] and tc5:
            ops.attention_tc5_diff(case.q_dev, out, i32(plan["pre"]), len(plan["pre"]) // 4, *seqs, *tail)
        elif plan["pre"]:
            ops.attention_diff_mma(case.q_dev, out, i32(plan["pre"]), len(plan["pre"]) // 2, *seqs, *tail)
        if plan["dec"]:
            n = len(plan["slots"]) // 2 * case.G * ops.DIFF_MAX_SPLITS * 2 * ops.DIFF_DECODE_ROWS
            part_o = torch.full((max(n, 1), case.vdim), float("nan"), device=DEV)
            part_ml = torch.full((max(n, 1), 2), float("nan"), device=DEV)
            ops.attention_diff_mma_decode(case.q_dev, out, i32(plan["dec"]), len(plan["dec"]) // 4, i32(plan["slots"] or [0]),
                                          len(plan["slots"]) // 2, part_o, part_ml, *seqs, *tail)
    ops.check_error_word(err)
    return out


DIFF_SHAPES = [  # lengths, query counts, H, G, dim, vdim, page, block of positions
    ((70, 33, 5, 129), (70, 1, 5, 2), 6, 2, 16, 40, 8, 20),
    ((100, 64, 17), (1, 64, 3), 4, 4, 24, 24, 16, 48),
    ((90, 40), (90, 1), 4, 1, 32, 32, 16, None),
    ((200, 131, 64, 65), (200, 1, 2, 65), 4, 2, 32, 64, 16, 64),
    ((300, 130), (172, 1), 2, 1, 64, 128, 16, 128),
    ((700, 300, 9), (700, 260, 9), 4, 2, 32, 64, 16, 256),
    ((1000, 40), (1000, 33), 8, 2, 64, 128, 32, None),
    # three query heads per kv head, pages of 8 and of 64; head sizes with swizzles of their own (16, 32) and the padded
    # ones (48, 80, 96, 112); the widest pair
    ((333, 150, 5), (333, 5, 5), 6, 2, 32, 64, 8, 96),
    ((260, 77), (260, 3), 3, 1, 64, 128, 64, 128),
    ((150, 70, 21), (150, 1, 4), 4, 2, 16, 32, 16, 48),
    ((150, 70, 21), (150, 1, 4), 2, 1, 48, 112, 16, 72),
    ((150, 70, 21), (150, 1, 4), 2, 2, 80, 112, 16, 100),
    ((200, 90), (200, 2), 2, 1, 128, 128, 16, None),
    ((130, 66), (130, 1), 2, 1, 16, 128, 16, 64),
    ((130, 66), (130, 1), 2, 1, 128, 16, 16, 64),
]


def kernels_for(dtype, dim, vdim, page=16):
    from mashbox_b200 import ops
    if dtype == "bfloat16" and ops.attention_tc5_diff_supports(dim, vdim, page):
        return ["simple", "mma", "mma-2", "mma-4", "mma-16", "tc5"]
    # the tensor-core kernels with the mixer's own plan, and with the short sequences cut into 2, 4 and 16 splits
    return ["simple"] + (["mma", "mma-2", "mma-4", "mma-16"] if dtype == "bfloat16" and ops.attention_diff_mma_supports(dim, vdim) else [])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", DIFF_SHAPES)
def test_differential_attention_kernels(dtype, shape):
    lengths, q_lens, H, G, dim, vdim, page, chunk = shape
    case = DiffCase(lengths, q_lens, H, G, dim, vdim, page, dtype, seed=len(lengths)).build()
    scale, lam, delta, eps = dim ** -0.5, 0.37, 0.28, 1e-5
    want = case.reference(scale, chunk, lam, delta, eps)
    for kernel in kernels_for(dtype, dim, vdim, page):
        kernel_close(run_diff(case, chunk, scale, lam, delta, eps, kernel), want, dtype, f"{kernel} kernel, {shape}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim,page,chunk", [(16, 40, 8, 20), (32, 64, 16, 64), (64, 128, 16, 128), (32, 32, 16, None)])
def test_one_loud_key_inside_and_outside_a_block(dtype, dim, vdim, page, chunk):
    """A key far louder than all others, placed at the first position of the query's block, at the last position of
    the block before, at the query's own position, at a page's first and last slot and (without a mask) hundreds of
    positions back: when the query may see it, the head's output is that key's value (up to the difference of the
    two maps and the norm); when it may not, the output is what it is without the loud key."""
    H, G = 4, 2
    block = chunk or 10 ** 9
    n = 3 * (chunk or 128) + 7
    for q_len in (1, 2, n):                                               # decoded alone, a short portion, a whole prompt
        pos = n - 1
        start = pos // block * block
        places = {start: True, pos: True, pos - 1: True}
        if chunk:
            places[start - 1] = False
            places[start - chunk] = False
        else:
            places[3] = True
        places[(pos // page) * page] = places.get((pos // page) * page, (pos // page) * page >= start)
        places[(pos // page) * page - 1] = places.get((pos // page) * page - 1, (pos // page) * page - 1 >= start)
        for place, seen in places.items():
            quiet = DiffCase((n,), (q_len,), H, G, dim, vdim, page, dtype, seed=11)
            loud = DiffCase((n,), (q_len,), H, G, dim, vdim, page, dtype, seed=11)
            # map 0 of kv head 0: the loud key is 8 times the last query of head 0 in map 0, normalised
            qv = loud.q[0][pos, 0, 0]
            loud.k[0][place, 0, 0] = (40.0 * qv / qv.norm() ** 2 / dim ** -0.5).to(TD[dtype]).double()
            quiet.build(), loud.build()
            for kernel in kernels_for(dtype, dim, vdim, page):
                a = run_diff(quiet, chunk, dim ** -0.5, 0.4, 0.2, 1e-6, kernel)[-1].float().cpu().reshape(H, vdim)
                b = run_diff(loud, chunk, dim ** -0.5, 0.4, 0.2, 1e-6, kernel)[-1].float().cpu().reshape(H, vdim)
                want = loud.reference(dim ** -0.5, chunk, 0.4, 0.2, 1e-6)[-1].reshape(H, vdim)
                kernel_close(b, want, dtype, f"{kernel}: loud key at {place}, query at {pos}, {q_len} queries")
                moved = float((a[0] - b[0]).abs().max())
                if seen:
                    assert moved > 0.05, f"{kernel}: the key at {place} must be seen from {pos} (block from {start})"
                else:
                    assert moved == 0.0, f"{kernel}: the key at {place} must not be seen from {pos} (block from {start})"


# ------------------------------------------------------------------------------------------------ the model in the engine
def runner_for(tmp, name, dtype, max_tokens, options=None, max_requests=4):
    from mashbox_b200.engine.replay import make_runner
    folder = L.make_folder(tmp, name, "float32" if dtype == "float32" else "bfloat16")
    return folder, make_runner(folder, dtype, max_tokens, page_size=L.CONFIGS[name][2], options=options,
                               max_requests=max_requests)


def replay(runner, steps):
    from mashbox_b200.engine.replay import run_step
    out = {}
    for i, s in enumerate(steps):
        r = run_step(runner, dict(s, step=i))
        if r is not None:
            out[i] = r.numpy()
    return out


def cut_steps(rid, tokens, cuts, end=True):
    """the steps that feed `tokens` in portions of the given sizes, asking for every position's logits"""
    steps, at = [], 0
    for n in cuts:
        steps.append(dict(entries=[dict(id=rid, tokens=tokens[at:at + n], want=list(range(n)))], end=[]))
        at += n
    assert at == len(tokens)
    if end:
        steps[-1]["end"] = [rid]
    return steps


CASES = [(n, d) for n in L.CONFIGS for d in DTYPES]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(tmp_path_factory, name, dtype):
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 320)
    for p in L.prompts_for(name, (1, 2, 3, 5, 21, 64, 65, 150, 300)):
        got = replay(runner, cut_steps("a", p, [len(p)]))[0]
        L.assert_close(got, L.plain_logits(folder, p), dtype, f"{name}: whole prompt of {len(p)}")
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.groups)


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(tmp_path_factory, name, dtype):
    """every token alone from the first one, over several blocks of positions and many pages, against the whole
    prompt in one step and against the plain implementation"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 192)
    (p,) = L.prompts_for(name, (170,), seed=1)
    whole = replay(runner, cut_steps("a", p, [len(p)]))[0]
    out = replay(runner, cut_steps("b", p, [1] * len(p)))
    single = np.concatenate([out[i] for i in range(len(p))])
    L.assert_close(single, L.plain_logits(folder, p), dtype, f"{name}: 170 tokens one by one")
    L.assert_close(single, whole, dtype, f"{name}: one by one against one step", L.BAR_SAME)
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 256)
    (p,) = L.prompts_for(name, (230,), seed=2)
    want = L.plain_logits(folder, p)
    whole = replay(runner, cut_steps("w", p, [len(p)]))[0]
    for cuts in ([2] * 115, [3, 37, 1, 2, 64, 17, 2, 2, 1, 50, 33, 5, 7, 6], [19, 20, 21, 1, 39, 40, 41, 49],
                 [63, 1, 1, 63, 2, 62, 38], [128, 2, 100]):
        out = replay(runner, cut_steps("a", p, cuts))
        got = np.concatenate([out[i] for i in range(len(cuts))])
        L.assert_close(got, want, dtype, f"{name}: portions {cuts[:6]}...")
        L.assert_close(got, whole, dtype, f"{name}: portions {cuts[:6]}... against one step", L.BAR_SAME)
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(tmp_path_factory, name, dtype):
    """Four requests at most are live, portions of some beside single tokens of others; the pool holds less than all
    requests together, and two state slots only, so pages and slots come back and are taken again.  Every request's
    logits must be those it has alone."""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 224, max_requests=2)
    prompts = dict(zip("abcdef", L.prompts_for(name, (90, 47, 3, 110, 66, 21), seed=3)))
    plans = dict(a=[30, 1, 1, 2, 50, 1, 1, 1, 1, 1, 1], b=[1, 1, 20, 2, 23], c=[1, 2], d=[64, 1, 40, 2, 1, 1, 1],
                 e=[2, 62, 1, 1], f=[21])
    order = ["a", "b", "c", "d", "e", "f"]
    at = {r: 0 for r in order}
    turn = {r: 0 for r in order}
    got = {r: [] for r in order}
    waiting, live, step = list(order), [], 0
    from mashbox_b200.engine.replay import run_step
    while waiting or live:
        while waiting and len(live) < 2:
            live.append(waiting.pop(0))
        entries, end = [], []
        for r in live:
            n = plans[r][turn[r]]
            entries.append(dict(id=r, tokens=prompts[r][at[r]:at[r] + n], want=list(range(n))))
            at[r] += n
            turn[r] += 1
            if turn[r] == len(plans[r]):
                assert at[r] == len(prompts[r])
                end.append(r)
        out = run_step(runner, dict(step=step, entries=entries, end=end)).numpy()
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
        live = [r for r in live if r not in end]
        runner.cache.check()
        step += 1
    for r in order:
        L.assert_close(np.concatenate(got[r]), L.plain_logits(folder, prompts[r]), dtype, f"{name}: request {r} in a batch")
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.groups)


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding_with_a_small_pool(tmp_path_factory, name, dtype):
    """a short prompt and 400 tokens one by one in a pool that holds them only because blocks that were left give
    their pages back (configurations whose every cache has a mask); two requests side by side, one a block ahead"""
    from mashbox_b200.config.registry import read_config
    from mashbox_b200.models.model import Model
    cfg = L.CONFIGS[name][0]
    entry, _ = read_config(cfg.to_hf())
    needs, _ = Model(entry.model_spec(cfg), cfg).cache_needs()
    masked = all(need.kind == "chunk" for need in needs.values())          # every cache gives left blocks back
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 448 if masked else 896)
    a, b = L.prompts_for(name, (412, 380), seed=4)
    steps = [dict(entries=[dict(id="a", tokens=a[:12], want=[11])], end=[]),
             dict(entries=[dict(id="a", tokens=a[12:44], want=[31]), dict(id="b", tokens=b[:3], want=[2])], end=[])]
    for i in range(400 - 32):
        e = [dict(id="a", tokens=[a[44 + i]], want=[0])]
        if 3 + i < len(b):
            e.append(dict(id="b", tokens=[b[3 + i]], want=[0]))
        steps.append(dict(entries=e, end=[]))
    out = replay(runner, steps)
    wa, wb = L.plain_logits(folder, a), L.plain_logits(folder, b)
    ga = np.stack([out[0][0], out[1][0]] + [out[2 + i][0] for i in range(368)])
    gb = np.stack([out[1][1]] + [out[2 + i][1] for i in range(368)])
    L.assert_close(ga, wa[[11, 43] + list(range(44, 412))], dtype, f"{name}: 368 tokens decoded, request a")
    L.assert_close(gb, wb[[2] + list(range(3, 371))], dtype, f"{name}: 368 tokens decoded, request b")
    if masked:
        assert max(max(runner.cache.pages_held(r)) for r in "ab") * runner.cache.page_size <= 2 * 128 + 32
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "float32"), ("R", "bfloat16")])
def test_greedy_generation_through_the_engine(tmp_path_factory, name, dtype):
    """Engine.generate with its scheduler, graphs and sampler: three prompts of unequal length in a pool too small for
    chunks of more than 32 tokens at once; in float32 the ids are the plain implementation's greedy ids."""
    from mashbox_b200.engine.engine import Engine
    folder = L.make_folder(tmp_path_factory.mktemp("m"), name, "float32" if dtype == "float32" else "bfloat16")
    eng = Engine.from_folder(folder, dtype=dtype, page_size=L.CONFIGS[name][2], max_tokens=512, max_requests=3, chunk=32,
                             max_tokens_per_step=40)
    prompts = L.prompts_for(name, (70, 5, 33), seed=5)
    new = 40
    r = eng.generate(prompts, max_new=new)
    assert r["finish"] == ["length"] * 3 and all(len(ids) == new for ids in r["ids"])
    again = eng.generate(prompts, max_new=new)                            # captured graphs now
    assert again["ids"] == r["ids"]
    assert eng.runner.stats["graph_replays"] > 0
    for p, ids in zip(prompts, r["ids"]):
        lg = L.plain_logits(folder, p + ids)
        for t, tok in enumerate(ids):
            row = lg[len(p) + t - 1]
            best = int(row.argmax())
            if dtype == "float32":
                assert tok == best or row[best] - row[tok] < 1e-4, f"{name}: token {t} is {tok}, plain says {best}"
            else:                                                          # bf16 may pick another of two near-equal ids
                assert row[best] - row[tok] < 0.05 * (row.max() - row.min()), f"{name}: token {t} = {tok} is far from the best"
    eng.cache.check()
