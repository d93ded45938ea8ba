"""Goguvik on the GPU against the plain statement: each mechanism alone, then the model through the
step function, the cache and the generation loop, cut into steps and batches in every way."""

import math

import pytest
import torch

import plain_goguvik as plain
from gpu_helpers import DTYPES, assert_close
from tiny import random_prompt
from tiny_goguvik import TINY_G, make_goguvik_folder

pytestmark = pytest.mark.gpu

CONFIGS = ["GA", "GB", "GC", "GD"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_cases, _runners = {}, {}


def case(tmp_path_factory, name, seed=1):
    if (name, seed) not in _cases:
        folder = make_goguvik_folder(tmp_path_factory.mktemp(f"g{name}{seed}"), name, seed=seed)
        _cases[(name, seed)] = (folder,) + plain.read_model_folder(folder)
    return _cases[(name, seed)]


def runner_for(tmp_path_factory, name, dtype, max_tokens=64 * 40):
    from starter_b200.engine import ModelRunner, load_model

    if (name, dtype) not in _runners:
        folder, _, _ = case(tmp_path_factory, name)
        _runners[(name, dtype)] = ModelRunner(load_model(folder, dtype), max_tokens=max_tokens, max_sequences=12)
    return _runners[(name, dtype)]


def close(got, want, dtype, what, fp32=2e-5, bf16=2e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = (fp32 if dtype in ("float32", torch.float32) else bf16) * float(want.abs().max())
    err = (got - want).abs()
    assert float(err.max()) <= tol, f"{what}: off by {float(err.max()):.3e} (allowed {tol:.3e}) at {tuple(int(i) for i in (err == err.max()).nonzero()[0])}"


# ------------------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_alone(dtype):
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, 72, generator=g, dtype=torch.float64) * 2
    d = torch.randn(9, 72, generator=g, dtype=torch.float64)
    alpha = torch.tensor(0.7, dtype=torch.float64)
    w, b = torch.randn(72, generator=g, dtype=torch.float64), torch.randn(72, generator=g, dtype=torch.float64)
    dev = lambda v, ty=torch.float32: v.to("cuda", ty).contiguous()  # noqa: E731
    xd, dd = dev(x, t), dev(d, t)
    args = (dev(alpha).reshape(1), dev(w), dev(b))
    close(ops.dynamic_tanh(xd, *args), plain.plain_dynamic_tanh(xd.double().cpu(), alpha, w, b), dtype, "norm alone")
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    both = (xd.double().cpu() + dd.double().cpu()).to(t).double()
    close(ops.dynamic_tanh(xd, *args, delta=dd, rows=rows), plain.plain_dynamic_tanh(both[[8, 0, 3]], alpha, w, b), dtype, "rows")
    assert torch.equal(xd, dev(x, t)), "selected rows must leave the stream alone"
    close(ops.dynamic_tanh(xd, *args, delta=dd), plain.plain_dynamic_tanh(both, alpha, w, b), dtype, "sum and norm")
    close(xd, both, dtype, "the sum is written back", bf16=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 37, 600])
@pytest.mark.parametrize("streams", [1, 2, 3, 4, 5, 8])
def test_stream_step_alone(streams, hidden, dtype):
    """The pending write, the next read and the norm in one kernel; the matrix is [from, to], every
    stream is formed from the OLD ones, and selected rows leave the streams as they were."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(10 + streams)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float64)  # noqa: E731
    x, y = rnd(7, streams, hidden), rnd(7, hidden)
    mix, out, read, bias = rnd(streams, streams), rnd(streams), rnd(streams), rnd(hidden)
    alpha, w, b = torch.tensor(0.4, dtype=torch.float64), rnd(hidden), rnd(hidden)
    dev = lambda v, ty=torch.float32: v.to("cuda", ty).contiguous()  # noqa: E731
    xd, yd = dev(x), dev(y, t)
    y_seen = yd.double().cpu()
    x_seen = xd.double().cpu()
    norm = (dev(alpha).reshape(1), dev(w), dev(b))
    new = plain.plain_stream_write(x_seen, y_seen + bias, mix, out)
    rows = torch.tensor([6, 2], dtype=torch.int32, device="cuda")
    # the model's end on selected rows: write, plain sum, norm; nothing stored
    got = ops.hyper_step(xd, t, (yd, dev(mix), dev(out), dev(bias)), None, norm, rows=rows)
    close(got, plain.plain_dynamic_tanh(new[[6, 2]].sum(1), alpha, w, b), dtype, "closing rows")
    assert torch.equal(xd, dev(x))
    # write, read, norm
    got = ops.hyper_step(xd, t, (yd, dev(mix), dev(out), dev(bias)), dev(read), norm)
    close(got, plain.plain_dynamic_tanh(plain.plain_stream_read(new, read), alpha, w, b), dtype, "write, read, norm")
    close(xd, new, "float32", "the streams after the write", fp32=1e-5)
    # a read with nothing pending and no norm
    got = ops.hyper_step(xd, t, None, dev(read), None)
    close(got, plain.plain_stream_read(xd.double().cpu(), read), dtype, "read alone")


def test_more_streams_than_the_kernel_takes_are_refused():
    from starter_b200 import ops

    x = torch.zeros(2, ops.max_streams() + 1, 8, device="cuda")
    with pytest.raises(ops.KernelError, match="streams"):
        ops.hyper_step(x, torch.float32, None, None, None)


def test_embedding_into_streams():
    from starter_b200 import ops

    table = torch.randn(11, 24, device="cuda").to(torch.bfloat16)
    tokens = torch.tensor([3, 10, 0], dtype=torch.int32, device="cuda")
    got = ops.embedding_streams(tokens, table, 3)
    assert got.dtype == torch.float32 and tuple(got.shape) == (3, 3, 24)
    for s in range(3):
        assert torch.equal(got[:, s], table[tokens.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [3, 40, 200, 600])
def test_gated_product_with_tanh_gelu(rows, dtype):
    """Every product kernel's gated epilogue knows the second activation (few rows, 128-row tiles, the
    library product followed by the activation kernel, the prompt product)."""
    from starter_b200 import ops

    t = TORCH[dtype]
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, 64, generator=g) * 1.5).to("cuda", t)
    w = (torch.randn(2 * 128, 64, generator=g) * 0.3).to("cuda", t)
    got = ops.linear(x, w, gated="gelu_tanh")
    xs, ws = x.double().cpu(), w.double().cpu()
    gate, up = xs @ ws[:128].T, xs @ ws[128:].T
    if dtype == "bfloat16":
        gate, up = gate.to(t).double(), up.to(t).double()
    close(got, plain.plain_gelu_tanh(gate) * up, dtype, f"{rows} rows", bf16=1.2e-2)
    silu = ops.linear(x, w, gated=True)
    close(silu, torch.nn.functional.silu(gate) * up, dtype, f"{rows} rows, silu as before", bf16=1.2e-2)


class Pages:
    """A cache by hand: one sequence whose pages are scattered, keys of both maps in one row."""

    def __init__(self, length, groups, dim, vdim, dtype, seed):
        g = torch.Generator().manual_seed(seed)
        self.k = torch.randn(length, groups, 2, dim, generator=g, dtype=torch.float64)
        self.v = torch.randn(length, groups, vdim, generator=g, dtype=torch.float64)
        self.length, self.groups, self.dim, self.vdim, self.t = length, groups, dim, vdim, TORCH[dtype]

    def store(self):
        n_pages = -(-self.length // 64)
        order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(5))[:n_pages]
        ks = torch.full((n_pages + 3, self.groups, 64, 2 * self.dim), 7.0, dtype=self.t, device="cuda")
        vs = torch.full((n_pages + 3, self.groups, 64, self.vdim), -9.0, dtype=self.t, device="cuda")
        for j in range(self.length):
            ks[order[j // 64], :, j % 64] = self.k[j].reshape(self.groups, -1).to("cuda", self.t)
            vs[order[j // 64], :, j % 64] = self.v[j].to("cuda", self.t)
        table = torch.zeros(2, n_pages, dtype=torch.int32, device="cuda")
        table[1] = order.to(torch.int32)
        self.k = torch.stack([ks[order[j // 64], :, j % 64].double().cpu().view(self.groups, 2, self.dim) for j in range(self.length)])
        self.v = torch.stack([vs[order[j // 64], :, j % 64].double().cpu() for j in range(self.length)])
        return ks, vs, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, dim, vdim", [(4, 2, 16, 24), (3, 3, 8, 40), (6, 1, 24, 16), (2, 1, 64, 128)])
def test_attention_alone_with_one_key_that_stands_out(heads, groups, dim, vdim, dtype):
    """Among 700 keys one is made to dominate map 1 and another map 2 (its query direction scaled up):
    far back, on either side of a page border, the newest.  A key that a kernel skips or reads from
    the wrong page changes the answer by the whole value."""
    from starter_b200 import ops

    t = TORCH[dtype]
    pages = Pages(700, groups, dim, vdim, dtype, seed=dim)
    ks, vs, table = pages.store()
    lam, lam0, eps, scale = 0.55, 0.3, 1e-5, 0.3
    for star1, star2 in ((2, 690), (63, 64), (64, 63), (699, 0), (127, 128), (640, 639)):
        for positions in ([699], [690, 691, 692, 693, 694, 695, 696, 697, 698, 699], [64, 63, 699, 128]):
            g = torch.Generator().manual_seed(star1)
            q = torch.randn(len(positions), heads, 2, dim, generator=g, dtype=torch.float64) * 0.3
            for h in range(heads):
                grp = h // (heads // groups)
                q[:, h, 0] += 6.0 * pages.k[star1, grp, 0] / scale / dim
                q[:, h, 1] += 6.0 * pages.k[star2, grp, 1] / scale / dim
            gate = torch.randn(len(positions), heads * vdim, generator=g, dtype=torch.float64)
            qd = q.reshape(len(positions), -1).to("cuda", t).contiguous()
            wide = torch.zeros(len(positions), heads * vdim + 5, dtype=t, device="cuda")   # a gate with a row stride
            wide[:, :heads * vdim] = gate.to("cuda", t)
            pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
            slot = torch.ones(len(positions), dtype=torch.int32, device="cuda")
            qs = qd.double().cpu().view(len(positions), heads, 2, dim)
            gs = wide[:, :heads * vdim].double().cpu()
            for warps in (1, 3, 8):
                got = ops.diff_attention(qd, wide[:, :heads * vdim], ks, vs, table, slot, pos, heads, groups, dim, vdim,
                                         scale, lam, 1 - lam0, eps, warps=warps)
                want = torch.cat([plain.plain_differential_head(
                    qs[:, h, 0], qs[:, h, 1], pages.k[:, h // (heads // groups), 0], pages.k[:, h // (heads // groups), 1],
                    pages.v[:, h // (heads // groups)], scale, lam, lam0, eps, torch.tensor(positions)) for h in range(heads)], -1)
                # a1 - lam * a2 cancels in part and the unit norm divides by what is left: float32 sums of
                # 64 products in the scores show up a few times larger than in the other tests
                close(got, want * torch.sigmoid(gs), dtype, f"keys {star1}/{star2}, queries at {positions}, {warps} warps",
                      fp32=1e-4)
    # a window: the key just inside is seen, the key just outside is not
    qd = torch.zeros(1, heads * 2 * dim, dtype=t, device="cuda")
    pos = torch.tensor([500], dtype=torch.int32, device="cuda")
    slot = torch.ones(1, dtype=torch.int32, device="cuda")
    got = ops.diff_attention(qd, None, ks, vs, table, slot, pos, heads, groups, dim, vdim, scale, 0.0, 1.0, 0.0, window=3)
    mean = pages.v[498:501].mean(0)
    want = torch.cat([mean[h // (heads // groups)] for h in range(heads)])
    want = (want.view(heads, vdim) / want.view(heads, vdim).pow(2).mean(-1, keepdim=True).sqrt()).reshape(1, -1)
    close(got, want, dtype, "a window of three keys")


@pytest.mark.parametrize("heads, groups, dim, vdim", [(4, 2, 16, 32), (2, 2, 32, 64), (3, 1, 64, 128), (2, 1, 128, 64),
                                                      (2, 1, 16, 128), (2, 2, 128, 128), (4, 2, 64, 64)])
def test_prompt_attention_on_tensor_cores_alone(heads, groups, dim, vdim):
    """Ragged sequences in one launch: a prompt from position 0, a portion that starts in the middle
    of a page behind 300 cached keys, a two-token portion; one key far back and one at the page
    border are made to stand out; with and without a window."""
    from starter_b200 import ops

    t = torch.bfloat16
    assert ops.diff_prefill_takes(t, dim, vdim)
    pages = Pages(700, groups, dim, vdim, "bfloat16", seed=dim + vdim)
    ks, vs, table = pages.store()
    lam, lam0, eps, scale = 0.45, 0.2, 1e-6, 0.25
    # (first position, count) per sequence; all read slot 1's pages, which is fine for reading
    spans = [(0, 150), (300, 333), (698, 2), (63, 66), (1, 128), (130, 129)]
    total = sum(n for _, n in spans)
    g = torch.Generator().manual_seed(7)
    q = torch.randn(total, heads, 2, dim, generator=g, dtype=torch.float64) * 0.3
    for h in range(heads):
        grp = h // (heads // groups)
        q[:, h, 0] += 5.0 * pages.k[3, grp, 0] / scale / dim
        q[:, h, 1] += 5.0 * pages.k[64, grp, 1] / scale / dim
    gate = torch.randn(total, heads * vdim, generator=g, dtype=torch.float64)
    qd = q.reshape(total, -1).to("cuda", t).contiguous()
    gd = gate.to("cuda", t).contiguous()
    qs, gs = qd.double().cpu().view(total, heads, 2, dim), gd.double().cpu()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    starts, at = [], 0
    for _, n in spans:
        starts.append(at)
        at += n
    tiles = [(i, f) for i, (_, n) in enumerate(spans) for f in range(0, n, 64)]
    for window in (None, 70):
        step = (i32([1] * len(spans)), i32(starts), i32([n for _, n in spans]), i32([p + n for p, n in spans]),
                i32([i for i, _ in tiles]), i32([f for _, f in tiles]))
        got = ops.diff_attention_prefill(qd, gd, ks, vs, table, *step, heads, groups, dim, vdim, scale, lam, 1 - lam0,
                                         eps, window, kernel="mma")
        kernels = [("mma.sync", got)]
        if ops.diff_prefill_tc_takes(t, dim, vdim):       # the same on the tcgen05 kernel
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            kernels.append(("tcgen05", ops.diff_attention_prefill(qd, gd, ks, vs, table, *step, heads, groups, dim, vdim,
                                                                  scale, lam, 1 - lam0, eps, window, status=status,
                                                                  kernel="tcgen05")))
            assert int(status.item()) == 0, "a wait inside the tcgen05 kernel ran out"
        for (p0, n), s0 in zip(spans, starts):
            positions = torch.arange(p0, p0 + n)
            want = torch.cat([plain.plain_differential_head(
                qs[s0:s0 + n, h, 0], qs[s0:s0 + n, h, 1], pages.k[:, h // (heads // groups), 0],
                pages.k[:, h // (heads // groups), 1], pages.v[:, h // (heads // groups)], scale, lam, lam0, eps,
                positions, window) for h in range(heads)], -1) * torch.sigmoid(gs[s0:s0 + n])
            for name, result in kernels:
                close(result[s0:s0 + n], want, "bfloat16", f"{name}: positions {p0}..{p0 + n - 1}, window {window}", bf16=2.5e-2)
        # the other kernel on the same rows agrees
        pos = i32([p for p0, n in spans for p in range(p0, p0 + n)])
        other = ops.diff_attention(qd, gd, ks, vs, table, i32([1] * total), pos, heads, groups, dim, vdim, scale, lam,
                                   1 - lam0, eps, window=window, warps=2)
        close(got, other, "bfloat16", f"both kernels, window {window}", bf16=2.5e-2)


@pytest.mark.parametrize("heads, groups, dim, vdim", [(4, 2, 16, 32), (2, 2, 32, 64), (8, 2, 64, 128), (2, 1, 128, 64),
                                                      (40, 2, 16, 128), (2, 2, 128, 128)])
def test_single_token_attention_on_tensor_cores_alone(heads, groups, dim, vdim):
    """Rows of unequal lengths in one launch (1 key, a page less one, a page, a page and one, 700),
    every number of parts from one to more than there are pages (up to eight joined inside a
    thread-block cluster, more, or all when told so, through scratch memory and a second kernel), a
    key far back and the newest made to stand out, with and without a window; 20 heads on one
    key/value head take two chunks of rows."""
    from starter_b200 import ops

    t = torch.bfloat16
    pages = Pages(700, groups, dim, vdim, "bfloat16", seed=3 * dim + vdim)
    ks, vs, table = pages.store()
    lam, lam0, eps, scale = 0.6, 0.25, 1e-6, 0.3
    lengths = [1, 63, 64, 65, 700, 130]
    g = torch.Generator().manual_seed(11)
    q = torch.randn(len(lengths), heads, 2, dim, generator=g, dtype=torch.float64) * 0.3
    for h in range(heads):
        grp = h // (heads // groups)
        q[:, h, 0] += 5.0 * pages.k[1, grp, 0] / scale / dim
        for r, n in enumerate(lengths):
            q[r, h, 1] += 5.0 * pages.k[n - 1, grp, 1] / scale / dim
    gate = torch.randn(len(lengths), heads * vdim, generator=g, dtype=torch.float64)
    qd, gd = q.reshape(len(lengths), -1).to("cuda", t).contiguous(), gate.to("cuda", t).contiguous()
    qs, gs = qd.double().cpu().view(len(lengths), heads, 2, dim), gd.double().cpu()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    for window in (None, 70):
        want = torch.stack([torch.cat([plain.plain_differential_head(
            qs[r:r + 1, h, 0], qs[r:r + 1, h, 1], pages.k[:, h // (heads // groups), 0], pages.k[:, h // (heads // groups), 1],
            pages.v[:, h // (heads // groups)], scale, lam, lam0, eps, torch.tensor([n - 1]), window)[0]
            for h in range(heads)]) for r, n in enumerate(lengths)]) * torch.sigmoid(gs)
        for splits, cluster in ((1, True), (1, False), (2, True), (3, True), (3, False), (5, True), (8, True),
                                (8, False), (11, True), (16, True), (None, True)):
            got = ops.diff_attention_decode(qd, gd, ks, vs, table, i32([1] * len(lengths)), i32(lengths), heads, groups,
                                            dim, vdim, scale, lam, 1 - lam0, eps, window, n_splits=splits, kv_hint=700,
                                            cluster=cluster)
            close(got, want, "bfloat16", f"{splits} parts, cluster {cluster}, window {window}", bf16=2.5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vdim", [12, 16])
def test_prepare_alone(vdim, dtype):
    """Biases, the temperature on both sides of every step of its quotient, and keys and values filed
    at their own places across a page border."""
    from starter_b200 import ops

    t = TORCH[dtype]
    heads, groups, dim, every, coef = 3, 1, 8, 8, 0.75      # value rows of 12 take the plain kernel, of 16 the vector one
    gate_w = heads * vdim
    width = heads * 2 * dim + gate_w + groups * (2 * dim + vdim)
    positions = [0, 6, 7, 8, 14, 15, 16, 62, 63, 64, 65, 127, 128]
    g = torch.Generator().manual_seed(1)
    proj = torch.randn(len(positions), width, generator=g).to("cuda", t)
    bias = torch.randn(width, generator=g).to("cuda")
    bias[heads * 2 * dim: heads * 2 * dim + gate_w] = 0
    ks = torch.zeros(5, groups, 64, 2 * dim, dtype=t, device="cuda")
    vs = torch.zeros(5, groups, 64, vdim, dtype=t, device="cuda")
    table = torch.tensor([[0, 0, 0], [4, 1, 3]], dtype=torch.int32, device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot = torch.ones(len(positions), dtype=torch.int32, device="cuda")
    q = ops.diff_prepare(proj, bias, heads, groups, dim, vdim, gate_w, (coef, every), pos, slot, table, ks, vs)
    full = proj.double().cpu() + bias.double().cpu()
    temp = plain.plain_query_temperature(torch.tensor(positions, dtype=torch.float64), coef, every)
    close(q, full[:, :heads * 2 * dim] * temp[:, None], dtype, "queries")
    k0 = heads * 2 * dim + gate_w
    for i, p in enumerate(positions):
        page = [4, 1, 3][p // 64]
        close(ks[page, :, p % 64].reshape(-1), full[i, k0:k0 + groups * 2 * dim], dtype, f"key at {p}")
        close(vs[page, :, p % 64].reshape(-1), full[i, k0 + groups * 2 * dim:], dtype, f"value at {p}")
    assert float(ks[0].abs().max()) == 0.0 and float(ks[2].abs().max()) == 0.0
    # a layer that only reads: queries (and gate) alone, nothing filed
    before = ks.clone()
    q2 = ops.diff_prepare(proj[:, :k0].contiguous(), bias[:k0].contiguous(), heads, groups, dim, vdim, gate_w, None,
                          pos, slot, table, None, None, write_cache=False)
    close(q2, full[:, :heads * 2 * dim], dtype, "queries without temperature")
    assert torch.equal(ks, before)


# ------------------------------------------------------------------------------ the model

def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    for length, seed in ((1, 1), (2, 2), (9, 3), (64, 4), (65, 5), (200, 6)):
        prompt = random_prompt(length, cfg["vocab"], seed)
        slot = runner.open_sequence()
        got = runner.step([StepEntry(slot, prompt, all_places(length))])
        runner.close_sequence(slot)
        want = plain.plain_forward(cfg, w, prompt)
        assert_close(got, want, dtype, f"{name} whole, length {length}")
        assert_close(got[:3], want[:3], dtype, f"{name}: the first tokens of a sequence")
    runner.check_status()
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_layer_against_the_plain_layers(tmp_path_factory, dtype):
    """The sum of the streams after each layer, which names the first layer that differs."""
    from starter_b200 import ops
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, "GA")
    runner = runner_for(tmp_path_factory, "GA", dtype)
    model = runner.model
    prompt = random_prompt(37, cfg["vocab"], 8)
    _, want = plain.plain_forward(cfg, w, prompt, return_layers=True)
    slot = runner.open_sequence()
    ctx = runner.make_context([StepEntry(slot, prompt, [])])
    streams = ops.embedding_streams(ctx.tokens, model.embed, model.spec.streams, ctx.status)
    pending = None
    rows = torch.arange(len(prompt), dtype=torch.int32, device="cuda")
    for i, entry in enumerate(model.spec.schedule):
        streams, pending = model.blocks[entry.layer](streams, pending, ctx, entry.cache, entry.writes_cache)
        total = ops.hyper_step(streams, torch.float32, (pending.value.float(),) + pending.for_kernel()[1:], None, None, rows=rows)
        close(total, want[i], dtype, f"after layer {i}", fp32=2e-5, bf16=2.5e-2)
    runner.close_sequence(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_prompt_then_tokens_one_by_one(tmp_path_factory, name, dtype):
    """The temperature's steps (every 8, 5, 48 or 16 positions) and a page border are crossed while decoding."""
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    for length, tail in ((40, 39), (100, 45), (150, 24)):
        prompt = random_prompt(length, cfg["vocab"], 10 + length)
        want = plain.plain_forward(cfg, w, prompt)
        slot = runner.open_sequence()
        head = length - tail
        rows = [runner.step([StepEntry(slot, prompt[:head], all_places(head))])]
        for tok in prompt[head:]:
            rows.append(runner.step([StepEntry(slot, [tok], [0])]))
        runner.close_sequence(slot)
        got = torch.cat(rows)
        assert_close(got, want, dtype, f"{name} last {tail} one by one, length {length}")
        assert_close(got[head:head + 1], want[head:head + 1], dtype, "the first single-token step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["GA", "GD"])
def test_long_decoding_over_many_pages(tmp_path_factory, name, dtype):
    """Two requests of unequal lengths decoded together for 420 steps: the longer one grows from one
    page to nine, so the single-token kernel goes from one part to several that join inside a cluster,
    and the shorter one ends on the way; every logit is held to the plain statement."""
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    lengths, heads = (560, 190), (140, 3)
    prompts = [random_prompt(n, cfg["vocab"], 300 + n) for n in lengths]
    want = [plain.plain_forward(cfg, w, p) for p in prompts]
    slots = [runner.open_sequence() for _ in prompts]
    first = runner.step([StepEntry(s, p[:h], all_places(h)) for s, p, h in zip(slots, prompts, heads)])
    got = [[first[:heads[0]]], [first[heads[0]:]]]
    at = list(heads)
    while at[0] < lengths[0]:
        live = [i for i in range(2) if at[i] < lengths[i]]
        rows = runner.step([StepEntry(slots[i], [prompts[i][at[i]]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(rows[k:k + 1])
            at[i] += 1
            if at[i] == lengths[i]:
                runner.close_sequence(slots[i])
    for i in range(2):
        assert_close(torch.cat(got[i]), want[i], dtype, f"{name} request {i} decoded to {lengths[i]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_portions_of_several_sizes(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    prompt = random_prompt(171, cfg["vocab"], 77)
    want = plain.plain_forward(cfg, w, prompt)
    for sizes in ((2, 2, 3, 57, 64, 1, 40, 2), (63, 2, 63, 43), (5, 128, 38)):
        slot = runner.open_sequence()
        rows, at = [], 0
        for n in sizes:
            rows.append(runner.step([StepEntry(slot, prompt[at:at + n], all_places(n))]))
            at += n
        assert at == len(prompt)
        runner.close_sequence(slot)
        assert_close(torch.cat(rows), want, dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_with_slots_and_pages_used_again(tmp_path_factory, name, dtype):
    from starter_b200.engine import StepEntry

    _, cfg, w = case(tmp_path_factory, name)
    runner = runner_for(tmp_path_factory, name, dtype)
    vocab = cfg["vocab"]
    batches = [[(70, 9), (5, 3), (33, 12), (1, 6)], [(2, 40), (129, 2), (64, 5)], [(17, 0), (63, 3)]]
    seed = 300
    for batch in batches:
        seqs, slots, got = [], [], []
        for plen, extra in batch:
            seed += 1
            seqs.append(random_prompt(plen + extra, vocab, seed))
            slots.append(runner.open_sequence())
            got.append([])
        first = runner.step([StepEntry(slots[i], seqs[i][:plen], all_places(plen)) for i, (plen, _) in enumerate(batch)])
        offset = 0
        for i, (plen, _) in enumerate(batch):
            got[i].append(first[offset:offset + plen])
            offset += plen
        live = [i for i, (_, extra) in enumerate(batch) if extra > 0]
        for i, (_, extra) in enumerate(batch):
            if extra == 0:
                runner.close_sequence(slots[i])
        step = 0
        while live:
            out = runner.step([StepEntry(slots[i], [seqs[i][batch[i][0] + step]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
            step += 1
            for i in [i for i in live if batch[i][1] == step]:
                runner.close_sequence(slots[i])
            live = [i for i in live if batch[i][1] > step]
        for i, seq in enumerate(seqs):
            assert_close(torch.cat(got[i]), plain.plain_forward(cfg, w, seq), dtype, f"{name} batch {batch}, request {i}")
        runner.cache.check()
    assert runner.cache.slots.held_count == 0 and runner.cache.pages.held_count == 0


@pytest.mark.parametrize("name", ["GA", "GC"])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name):
    """Unequal prompts through ``Engine.generate`` (the scheduler, the captured single-token step, the
    sampler): 70 tokens each, past a page border and several temperature steps, equal to the plain
    statement's greedy continuation."""
    from starter_b200 import Engine

    folder, cfg, w = case(tmp_path_factory, name)
    engine = Engine(folder, dtype="float32", max_batch=4)
    prompts = [random_prompt(n, cfg["vocab"], 900 + n) for n in (50, 3, 21)]
    steps = list(engine.generate(prompts, 70))
    assert len(steps) == 70
    for i, prompt in enumerate(prompts):
        assert [s[i] for s in steps] == plain.plain_generate(cfg, w, prompt, 70), f"request {i}"


def test_random_weights_from_the_library_run_in_bfloat16(tmp_path_factory):
    """``random_model`` places every tensor as the loader would, and sampling with temperature runs."""
    from starter_b200 import Engine
    from starter_b200.config import config_from_dict
    from starter_b200.engine.runner import random_model

    model = random_model(config_from_dict(TINY_G["GA"]), seed=5, dtype="bfloat16")
    engine = Engine.from_model(model, max_batch=2)
    out = engine.complete([[1, 2, 3], [4]], 12, temperature=0.8, seed=3)
    assert [len(c.tokens) for c in out] == [12, 12]
    assert all(0 <= t < 200 for c in out for t in c.tokens)


# ------------------------------------------------------------------------------ the programs

def test_command_line_and_trace_replay(tmp_path_factory, tmp_path):
    """``python -m starter_b200 generate`` and ``bin/trace_run`` pick the design by its config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, cfg, w = case(tmp_path_factory, "GD")
    prompts = [random_prompt(5, cfg["vocab"], 1), random_prompt(19, cfg["vocab"], 2)]
    text = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model-path", folder, "--input-ids", text,
                          "--max-new-tokens", "6", "--dtype", "float32"], cwd=root, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    assert [line["tokens"] for line in lines] == [plain.plain_generate(cfg, w, p, 6) for p in prompts]
    out = subprocess.run([sys.executable, "-m", "starter_b200", "generate", "--model-path", folder, "--prompt-lens", "4,2",
                          "--max-new-tokens", "3"], cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr

    # a trace: two unequal requests start together, are decoded together, the shorter one ends first
    a, b = random_prompt(140, cfg["vocab"], 5), random_prompt(70, cfg["vocab"], 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:130], "want": [0, 129]},
                                     {"id": "b", "tokens": b[:66], "want": [65]}], "end": []}]
    for i in range(10):
        entries = [{"id": "a", "tokens": [a[130 + i]], "want": [0]}]
        if i < 4:
            entries.append({"id": "b", "tokens": [b[66 + i]], "want": [0] if i % 2 else []})
        steps.append({"step": 1 + i, "entries": entries, "end": (["b"] if i == 3 else []) + (["a"] if i == 9 else [])})
    for dtype in DTYPES:
        out_dir = str(tmp_path / dtype)
        proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                                 "--out", out_dir, "--max-tokens", "210"], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                text=True)
        for record in steps:
            proc.stdin.write(json.dumps(record) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {record['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
        want_a, want_b = plain.plain_forward(cfg, w, a), plain.plain_forward(cfg, w, b)
        read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))  # noqa: E731
        assert_close(read(0), torch.stack([want_a[0], want_a[129], want_b[65]]), dtype, "the first step")
        for i in range(10):
            rows = [want_a[130 + i]] + ([want_b[66 + i]] if i < 4 and i % 2 else [])
            assert_close(read(1 + i), torch.stack(rows), dtype, f"step {1 + i}")
