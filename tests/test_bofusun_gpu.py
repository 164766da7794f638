"""The Bofusun decoder in the engine against the plain statement of its equations.

Kernels and parts alone; whole prompts; token-by-token decoding; portions down to two tokens;
unequal requests in one batch against each alone; rows and pages that are used again; keys far
back, at page borders and on both sides of a window's edge, in prompts and decoded; weights made
so that one far key or one key at the window's edge decides the result; greedy generation through
the engine's entry point and scheduler; a replay through bin/trace_run.
"""

import numpy as np
import pytest
import torch

import plain_bofusun as plain
from bofusun_tiny import TINY, Harness, make_folder, rel_err
from traces import Trace, compare, last_decoded, mixed, portions, run_trace, whole

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------
# kernels alone

def test_fold_rmsnorm_kernel():
    from socrates_b200.kernels import ops
    g = torch.Generator(device=DEV).manual_seed(0)
    N, d, S = 7, 52, 3
    res = torch.randn(N, d, device=DEV, generator=g)
    delta = torch.randn(S, N, d, device=DEV, generator=g)
    bias, bgain, gain, vec = (torch.randn(d, device=DEV, generator=g) for _ in range(4))
    rows = torch.randn(N, d, device=DEV, generator=g)
    for out_dtype in (torch.float32, torch.bfloat16):
        for use in range(16):
            kw = dict(branch_bias=bias if use & 1 else None, branch_gain=bgain if use & 2 else None,
                      branch_eps=1e-3, add_rows=rows if use & 4 else None, add_vec=vec if use & 8 else None)
            r = res.clone()
            out = torch.empty(N, d, device=DEV, dtype=out_dtype)
            ops.fold_rmsnorm(r, delta, gain, out, 1e-5, **kw)
            b = delta.double().sum(0) + (bias.double() if use & 1 else 0)
            if use & 2:
                b = plain.unit_rms(b, 1e-3) * bgain.double()
            v = res.double() + b + (rows.double() if use & 4 else 0) + (vec.double() if use & 8 else 0)
            assert torch.allclose(r.double(), v, atol=1e-5)
            want = plain.unit_rms(v, 1e-5) * gain.double()
            assert torch.allclose(out.double(), want, atol=1e-5 if out_dtype == torch.float32 else 3e-2, rtol=1e-2)
    # only some rows, nothing written back; and a fold without an output
    r = res.clone()
    idx = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(3, d, device=DEV)
    ops.fold_rmsnorm(r, delta, gain, out, 1e-5, idx, branch_gain=bgain, branch_eps=1e-3)
    v = res.double() + plain.unit_rms(delta.double().sum(0), 1e-3) * bgain.double()
    assert torch.equal(r, res)
    assert torch.allclose(out.double(), (plain.unit_rms(v, 1e-5) * gain.double())[idx.long()], atol=1e-5)
    ops.fold_rmsnorm(r, delta, None, None, 0.0, branch_gain=bgain, branch_eps=1e-3)
    assert torch.allclose(r.double(), v, atol=1e-5)


def test_normed_mean_and_bias_act_kernels():
    from socrates_b200.kernels import ops
    g = torch.Generator(device=DEV).manual_seed(1)
    N, d = 5, 44
    a, b = torch.randn(2, N, d, device=DEV, generator=g), torch.randn(1, N, d, device=DEV, generator=g) * 30
    ga, gb = torch.randn(d, device=DEV, generator=g), torch.randn(d, device=DEV, generator=g)
    out = torch.empty(N, d, device=DEV)
    ops.normed_mean(out, a, ga, b, gb, 1e-4, 0.5)
    want = 0.5 * (plain.unit_rms(a.double().sum(0), 1e-4) * ga.double() + plain.unit_rms(b.double()[0], 1e-4) * gb.double())
    assert torch.allclose(out.double(), want, atol=1e-5)
    x = torch.randn(N, d, device=DEV, generator=g) * 2
    bias = torch.randn(d, device=DEV, generator=g)
    acts = {"relu_squared": lambda z: torch.relu(z) ** 2, "gelu_tanh": plain.gelu_tanh, "silu": plain.silu,
            "identity": lambda z: z}
    for name, fn in acts.items():
        y = torch.empty(N, d, device=DEV)
        ops.bias_act(y, x, bias, name)
        assert torch.allclose(y.double(), fn(x.double() + bias.double()), atol=1e-5), name
        parts = torch.stack([x * 0.25, x * 0.75])
        yb = torch.empty(N, d, device=DEV, dtype=torch.bfloat16)
        ops.bias_act(yb, parts, None, name)
        assert torch.allclose(yb.double(), fn(x.double()), atol=3e-2, rtol=2e-2), name


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("dtype", DTYPES)
def test_short_conv_in_portions(taps, dtype):
    """Three sequences of unequal length, cut at different places (portions of one and two tokens, shorter
    than the taps), share the steps; the tails carry what each portion's first tokens need."""
    from socrates_b200.kernels import ops
    g = torch.Generator().manual_seed(taps)
    C, lengths = 21, [19, 7, 30]
    u = [torch.randn(n, C + 3, generator=g).to(dtype) for n in lengths]
    w, b_in, b_conv = torch.randn(C, taps, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    want = [plain.silu(plain.short_conv(x[:, :C].double() + b_in.double(), w.double(), b_conv.double())) for x in u]
    tail = torch.zeros(5, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    if tail is not None:
        tail = tail[:, :taps - 1].contiguous()
        tail += 7.0                                     # what a previous owner left in the slots ...
        tail[[4, 0, 2]] = 0.0                           # ... and the rows of this test, as `assign` leaves them
    rows = [4, 0, 2]
    cuts = [[1, 2, 1, 5, 10], [2, 1, 1, 1, 2], [6, 1, 2, 20, 1]]
    got = [[] for _ in lengths]
    fed = [0, 0, 0]
    for step in range(5):
        batch = [(i, cuts[i][step]) for i in range(3) if fed[i] < lengths[i]]
        x = torch.cat([u[i][fed[i]:fed[i] + c] for i, c in batch]).to(DEV).contiguous()
        token_rows = torch.tensor([rows[i] for i, c in batch for _ in range(c)], dtype=torch.int32, device=DEV)
        pos = torch.tensor([fed[i] + t for i, c in batch for t in range(c)], dtype=torch.int32, device=DEV)
        starts = torch.tensor(np.cumsum([0] + [c for _, c in batch]), dtype=torch.int32, device=DEV)
        seq_rows = torch.tensor([rows[i] for i, _ in batch], dtype=torch.int32, device=DEV)
        y = torch.empty(x.shape[0], C, device=DEV, dtype=dtype)
        ops.short_conv(x, b_in.to(DEV), w.to(DEV), b_conv.to(DEV), True, tail, token_rows, pos, [(0, C, y)])
        if tail is not None:
            ops.short_conv_tail(tail, x, b_in.to(DEV), taps, starts, seq_rows)
        o = 0
        for i, c in batch:
            got[i].append(y[o:o + c].double().cpu())
            o += c
            fed[i] += c
    for i in range(3):
        mine = torch.cat(got[i])
        assert mine.shape[0] == lengths[i]
        assert torch.allclose(mine, want[i], atol=1e-5 if dtype == torch.float32 else 5e-2, rtol=2e-2)


# ------------------------------------------------------------------------------------------
# parts alone: a mixer fed a sequence in portions equals the plain function on the whole

def mixer_in_portions(tmp_path, name, dtype, entry, sizes, n, plain_fn):
    from socrates_b200.engine.context import CacheView
    from socrates_b200.engine.runner import StepEntry
    folder, cfg, w = make_folder(tmp_path, name)
    h = Harness(folder, dtype, max_len=640)
    layer = h.model.plan.order[entry].layer
    mixer = h.model.layers[layer].mixer
    g = torch.Generator().manual_seed(entry + n)
    x = (torch.randn(n, cfg["width"], generator=g) * 1.5).to(dtype)
    want = plain_fn(x.double(), w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], cfg["norm"]["eps"])
    h.cache.assign(2)
    got, start, k = [], 0, 0
    while start < n:
        c = min(sizes[min(k, len(sizes) - 1)], n - start)
        assert h.cache.reserve(2, start + c)
        ctx = h.runner.prepare([StepEntry(2, [0] * c, start, [c - 1])])
        branch = mixer.forward(ctx, x[start:start + c].to(DEV).contiguous(), CacheView(h.cache, entry, True))
        got.append(branch.partial.sum(0).double().cpu())
        h.cache.commit(2, start + c)
        start, k = start + c, k + 1
    got = torch.cat(got)
    scale = float(want.abs().max())
    return float((got - want).abs().max()) / scale


PART_TOL = {torch.float32: 5e-5, torch.bfloat16: 4e-2}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(150,), (1,), (2,), (40, 3, 1, 2, 70, 1)])
@pytest.mark.parametrize("name,entry", [("P", 0), ("P", 6), ("Q", 1), ("R", 1)])
def test_retention_part(tmp_path, dtype, sizes, name, entry):
    err = mixer_in_portions(tmp_path, name, dtype, entry, sizes, 150, plain.retention)
    assert err < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(90,), (1,), (2,), (15, 2, 1, 1, 30, 17, 3)])
@pytest.mark.parametrize("name,entry", [("P", 1), ("Q", 0), ("R", 0), ("R", 2)])
def test_parallel_part(tmp_path, dtype, sizes, name, entry):
    """Windowed attention beside the selective scan, normed and averaged; 90 tokens pass every window's
    edge and several page borders, in one portion, token by token and in ragged portions."""
    err = mixer_in_portions(tmp_path, name, dtype, entry, sizes, 90, plain.parallel_mixer)
    assert err < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(600,), (290, 1, 309), (64, 2, 400, 134)])
@pytest.mark.parametrize("name,entry", [("P", 0), ("P", 1), ("R", 2)])
def test_long_portions(tmp_path, dtype, sizes, name, entry):
    """Portions of hundreds of tokens: retention in chunks and the scan in segments that run side by side
    (scratch states, a scan over them), attention far past its window, against the same plain functions."""
    layer_type = TINY[name][0]["layers"][{0: 0, 1: 1, 2: 2}[entry] if name == "P" else 2]["type"]
    fn = plain.retention if layer_type == "retention" else plain.parallel_mixer
    err = mixer_in_portions(tmp_path, name, dtype, entry, sizes, 600, fn)
    assert err < PART_TOL[dtype] * 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_inner_mixers_alone(tmp_path, dtype):
    """The two halves of a parallel mixer each against its own plain function."""
    from socrates_b200.engine.context import CacheView
    from socrates_b200.engine.runner import StepEntry
    folder, cfg, w = make_folder(tmp_path, "R")
    h = Harness(folder, dtype, max_len=256)
    n = 70
    x = (torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(5)) * 1.5).to(dtype)
    pair = h.model.layers[0].mixer
    m = cfg["layers"][0]["mixer"]
    want = [plain.gated_window_attention(x.double(), w, "l0.mix.left.", m["left"]),
            plain.selective_scan(x.double(), w, "l0.mix.right.", m["right"])]
    h.cache.assign(0)
    got = [[], []]
    for start, c in ((0, 33), (33, 1), (34, 36)):
        assert h.cache.reserve(0, start + c)
        ctx = h.runner.prepare([StepEntry(0, [0] * c, start, [c - 1])])
        view = CacheView(h.cache, 0, True)
        for i, (pre, inner) in enumerate(zip(pair.prefixes, pair.inner)):
            got[i].append(inner.forward(ctx, x[start:start + c].to(DEV).contiguous(), view.sub(pre)).partial.sum(0).double().cpu())
        h.cache.commit(0, start + c)
    for i in range(2):
        mine = torch.cat(got[i])
        assert float((mine - want[i]).abs().max() / want[i].abs().max()) < PART_TOL[dtype], i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_stream_after_every_layer_run(tmp_path, dtype, name):
    """The residual stream after every run of a layer (repeated layers count each time): the embedding's
    norm, the norms on both sides of each branch, the additions at the start of a pass."""
    import socrates_b200.engine.context as C
    from socrates_b200.parts.norm import fold_and_norm
    folder, cfg, w = make_folder(tmp_path, name)
    ids = tokens(cfg["vocab"], 45, 11)
    want = []
    plain.forward(cfg, w, ids, want)
    h = Harness(folder, dtype)
    got = []

    def after(i, stream):
        fold_and_norm(stream, None, None, 0.0)
        got.append(stream.residual.double().cpu())

    original = C.StepContext.__init__

    def patched(self, *a, **k):
        original(self, *a, **k)
        self.after_run = after
    C.StepContext.__init__ = patched
    try:
        h.step([("a", ids)])
    finally:
        C.StepContext.__init__ = original
    assert len(got) == len(want) == len(h.model.plan.order)
    for i, (a, b) in enumerate(zip(got, want)):
        assert float((a - b).abs().max() / b.abs().max()) < (1e-4 if dtype == torch.float32 else 8e-2), i


# ------------------------------------------------------------------------------------------
# whole models

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("bofusun")
    out = {}
    for name in TINY:
        folder, cfg, w = make_folder(tmp, name)
        seqs = [tokens(cfg["vocab"], n, 50 + i) for i, n in enumerate((150, 23, 77, 4))]
        out[name] = (folder, cfg, w, seqs, [plain.forward(cfg, w, s) for s in seqs])
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompts_decoding_and_portions(models, dtype, name):
    folder, cfg, w, seqs, want = models[name]
    h = Harness(folder, dtype)
    ids, ref = seqs[0], want[0]
    ways = {"whole": h.run("w", ids, (len(ids),)),
            "token by token": h.run("d", ids, (1,)),
            "pairs": h.run("p", ids, (2,)),
            "ragged": h.run("r", ids, (7, 2, 16, 3, 2, 33, 5, 17, 2, 1, 1, 1, 40)),
            "prompt then decoded": h.run("t", ids, (len(ids) - 40, 1))}
    for way, got in ways.items():
        assert rel_err(got, ref) < TOL[dtype], way
    if dtype == torch.float32:          # how the tokens were cut changes rounding only
        for way, got in ways.items():
            assert rel_err(got, ways["whole"]) < 2e-5, way
    # the first tokens of a sequence, alone
    assert rel_err(h.run("f", seqs[3], (1,)), want[3]) < TOL[dtype]
    assert rel_err(h.run("g", seqs[3], (4,)), want[3]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S"])
def test_unequal_requests_in_one_batch(models, dtype, name):
    """Four requests of 150, 23, 77 and 4 tokens: portions of some beside single tokens of others, a
    request that joins late and one that sits steps out; each must come out as it does alone."""
    folder, cfg, w, seqs, want = models[name]
    h = Harness(folder, dtype)
    alone = [Harness(folder, dtype).run("x", s, (len(s),)) for s in seqs] if dtype == torch.float32 else None
    fed = [0] * 4
    got = [[] for _ in seqs]
    plan = [[(0, 60), (1, 1)], [(0, 1), (1, 1), (2, 30)], [(0, 2), (2, 1), (3, 4)], [(1, 20), (2, 1)],
            [(0, 30), (1, 1), (2, 44)], [(0, 1), (2, 1)], [(0, 56)]]
    for step in plan:
        entries = [(f"r{i}", seqs[i][fed[i]:fed[i] + c]) for i, c in step if fed[i] < len(seqs[i])]
        ended = [f"r{i}" for i, c in step if fed[i] < len(seqs[i]) and fed[i] + c >= len(seqs[i])]
        out = h.step(entries, end=ended)
        for i, c in step:
            if f"r{i}" in out:
                got[i].append(out[f"r{i}"])
                fed[i] += out[f"r{i}"].shape[0]
    for i, s in enumerate(seqs):
        mine = torch.cat(got[i])
        assert mine.shape[0] == len(s)
        assert rel_err(mine, want[i]) < TOL[dtype], i
        if alone is not None:
            assert rel_err(mine, alone[i]) < 2e-5, i


@pytest.mark.parametrize("dtype", DTYPES)
def test_rows_and_pages_are_used_again(models, dtype):
    """Two rows and a pool of 12 pages of 16 slots serve eight requests one after another, in portions
    and token by token: every state slot and page is handed out several times, dirty from its previous owner."""
    folder, cfg, w, seqs, want = models["P"]
    h = Harness(folder, dtype, max_rows=2, max_len=160, pages=12)
    order = [0, 1, 2, 3, 2, 0, 3, 1]
    for k in range(0, len(order), 2):
        a, b = order[k], order[k + 1]
        ga = h.run(f"a{k}", seqs[a], (31, 1, 2, 64))
        fed, gb = 0, []
        while fed < len(seqs[b]):                       # the second of the pair decodes token by token
            gb.append(h.step([(f"b{k}", seqs[b][fed:fed + 1])], end=[f"b{k}"] if fed + 1 == len(seqs[b]) else [])[f"b{k}"])
            fed += 1
        assert rel_err(ga, want[a]) < TOL[dtype] and rel_err(torch.cat(gb), want[b]) < TOL[dtype], k
    assert h.cache.free_pages() == [12]


def plant(folder, w, q_name, k_name, rows, x_query, x_key, boost):
    """Make one (query, key) pair stand out: the query projection gets a large component along the input
    `x_query` and the key projection along `x_key`, in the head dims `rows`.  Rewrites the folder's weights."""
    from safetensors.torch import save_file
    w = dict(w)
    wk, wq = w[k_name].clone(), w[q_name].clone()
    wk[rows] += boost * x_key / x_key.norm()
    wq[rows] += boost * x_query / x_query.norm()
    w[k_name], w[q_name] = wk.bfloat16().double(), wq.bfloat16().double()
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return w


def _planted(folder, cfg, w, layer_prefix, q_name, k_name, rows, key_token, query_token, boost):
    """`plant` for the first layer of a model: the inputs are those of two token ids."""
    eps = cfg["norm"]["eps"]
    e = plain.norm_around_zero(w["embed"], w["embed.norm"], eps)
    if "loop" in cfg and cfg["loop"]["start"] == 0:
        e = e + w["loop.step"][0]
    x = plain.norm_around_zero(e, w[layer_prefix + "norm1"], eps)
    return plant(folder, w, q_name, k_name, rows, x[query_token], x[key_token], boost)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_decides_retention(tmp_path, dtype):
    """The retention part alone: among 440 keys the one at position 3, planted in the dims that do not
    rotate of the head with the slowest decay, is most of what the last queries read.  Losing it, or
    decaying it by one step too many or too few, changes the part's output by far more than the tolerance."""
    from socrates_b200.engine.context import CacheView
    from socrates_b200.engine.runner import StepEntry
    folder, cfg, w = make_folder(tmp_path, "P")
    n = 440
    x = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(8)) * 1.5
    u = x[3] / x[3].norm()
    keep = x[3].clone()
    x = x - (x @ u)[:, None] * u[None, :]          # no other input has a component along the planted key's
    x[3] = keep
    x = x.bfloat16().double()
    for p in (403, 420):
        x[p] = x[439]
    rows = [2 * 8 + 4, 2 * 8 + 5, 2 * 8 + 6, 2 * 8 + 7]           # head 2, dims 4..7 (rot.dims = 4)
    w = plant(folder, w, "l0.mix.q", "l0.mix.k", rows, x[439], x[3], 40.0)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    want = plain.retention(x, w, "l0.mix.", m, eps)
    lost = x.clone()
    lost[3] = x[4]
    assert float((plain.retention(lost, w, "l0.mix.", m, eps)[439] - want[439]).abs().max() / want.abs().max()) > 0.3
    for sizes in ((n,), (400, 1), (100, 2, 250, 50, 1)):
        h = Harness(folder, dtype, max_len=448)
        mixer = h.model.layers[0].mixer
        h.cache.assign(1)
        got, start, k = [], 0, 0
        while start < n:
            c = min(sizes[min(k, len(sizes) - 1)], n - start)
            assert h.cache.reserve(1, start + c)
            ctx = h.runner.prepare([StepEntry(1, [0] * c, start, [c - 1])])
            xin = x[start:start + c].to(torch.float32 if dtype == torch.float32 else torch.bfloat16).to(DEV).contiguous()
            got.append(mixer.forward(ctx, xin, CacheView(h.cache, 0, True)).partial.sum(0).double().cpu())
            h.cache.commit(1, start + c)
            start, k = start + c, k + 1
        assert float((torch.cat(got) - want).abs().max() / want.abs().max()) < PART_TOL[dtype], sizes


@pytest.mark.parametrize("dtype", [torch.float32])
def test_one_far_key_decides(tmp_path, dtype):
    """The whole model P in float32 (where the tolerance is far below what the key contributes): one key
    400 tokens back, planted in layer 0's retention, shows in the last logits.  Whole, and with the tail
    decoded.  Both dtypes are covered on the part alone, above."""
    folder, cfg, w = make_folder(tmp_path, "P")
    key_tok, query_tok = 5, 9
    rows = [2 * 8 + 4, 2 * 8 + 5, 2 * 8 + 6, 2 * 8 + 7]           # head 2, dims 4..7 (rot.dims = 4)
    w = _planted(folder, cfg, w, "l0.", "l0.mix.q", "l0.mix.k", rows, key_tok, query_tok, 6.0)
    others = [t for t in range(cfg["vocab"]) if t not in (key_tok, query_tok)]
    g = torch.Generator().manual_seed(2)
    ids = [others[int(i)] for i in torch.randint(0, len(others), (440,), generator=g)]
    ids[3] = key_tok
    for p in (403, 420, 439):
        ids[p] = query_tok
    ref = plain.forward(cfg, w, ids)
    without = list(ids)
    without[3] = others[0]
    assert rel_err(plain.forward(cfg, w, without)[439:], ref[439:]) > 0.003     # the far key shows in the logits
    h = Harness(folder, dtype, max_len=448)
    assert rel_err(h.run("a", ids, (440,)), ref) < TOL[dtype]
    assert rel_err(h.run("b", ids, (400, 1)), ref) < TOL[dtype]
    assert rel_err(h.run("c", ids, (100, 2, 250, 50, 1)), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_key_at_the_windows_edge_decides(tmp_path, dtype):
    """Windowed attention, layer 0 of Q (one tap, no cap, a window of 37): a key with a very large score
    is seen by the query 36 tokens later and not by the one 37 later.  In a prompt, decoded, and with the
    key in an earlier portion; the key sits on the last slot of a page in one run and the first in another."""
    folder, cfg, w = make_folder(tmp_path, "Q")
    key_tok, query_tok = 7, 11
    w = _planted(folder, cfg, w, "l0.", "l0.mix.left.q", "l0.mix.left.k", list(range(16)), key_tok, query_tok, 9.0)
    others = [t for t in range(cfg["vocab"]) if t not in (key_tok, query_tok)]
    g = torch.Generator().manual_seed(3)
    # the planted scores are large, and bfloat16 rounds them coarsely; a key wrongly seen or lost moves the logits by 0.5 and more
    tol = TOL[dtype] if dtype == torch.float32 else 0.15
    for key_at in (15, 16, 40):
        ids = [others[int(i)] for i in torch.randint(0, len(others), (key_at + 60,), generator=g)]
        ids[key_at] = key_tok
        ids[key_at + 36] = query_tok          # the last query that sees the key
        ids[key_at + 37] = query_tok          # the first that does not
        ref = plain.forward(cfg, w, ids)
        assert rel_err(ref[key_at + 36], ref[key_at + 37]) > 0.5           # the edge shows in the logits
        h = Harness(folder, dtype)
        assert rel_err(h.run("a", ids, (len(ids),)), ref) < tol, key_at
        assert rel_err(h.run("b", ids, (key_at + 20, 1)), ref) < tol, key_at
        assert rel_err(h.run("c", ids, (key_at + 1, 35, 2, 1)), ref) < tol, key_at
        assert rel_err(h.run("d", ids, (key_at + 36, 2, 1)), ref) < tol, key_at


# ------------------------------------------------------------------------------------------
# the entry point, the scheduler, the command-line replay

@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", True)])
@pytest.mark.parametrize("name", ["P", "R", "S"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, graphs):
    """Five requests through Engine: queued, admitted as rows come free, prompts cut by the token
    budget, decoded side by side (bfloat16: through recorded graphs), 90 new tokens each, which passes
    every window.  Every produced token is the plain statement's choice, or within its margin."""
    from socrates_b200 import Engine
    folder, cfg, w, seqs, _ = models[name]
    prompts = [seqs[0][:70], seqs[1], seqs[2][:40], seqs[3], seqs[0][70:101]]
    eng = Engine(str(folder), device="cuda:0", dtype=dtype, compile=graphs, max_batch=3, max_len=192,
                 max_new_tokens=90, token_budget=48)
    reqs = [eng.submit(p) for p in prompts]
    while eng.scheduler.has_work():
        assert eng.step()
        eng.scheduler.check()
    margin = 1e-3 if dtype == "float32" else 8e-2
    for p, r in zip(prompts, reqs):
        assert r.done and len(r.output) == 90
        logits = plain.forward(cfg, w, list(p) + r.output[:-1])
        scale = float(logits.abs().max())
        for i, tok in enumerate(r.output):
            row = logits[len(p) - 1 + i]
            best = int(torch.argmax(row))
            assert tok == best or float(row[best] - row[tok]) <= margin * scale, (i, tok, best)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(models, tmp_path, dtype):
    """bin/trace_run on model R: whole, tail decoded, portions, and a mix of up to four live requests
    in a pool that only holds the busiest step."""
    folder, cfg, w, seqs, want = models["R"]
    named = {f"s{i}": s for i, s in enumerate(seqs[:3])}
    reference = {k: want[i].numpy() for i, k in enumerate(named)}
    trace = Trace()
    for k, ids in named.items():
        whole(trace, "w:" + k, ids)
        last_decoded(trace, "d:" + k, ids, tail=20)
        portions(trace, "p:" + k, ids)
    mixed(trace, {f"m{j}:{k}": ids for j in range(2) for k, ids in named.items()}, seed=5, tail=20)
    result = run_trace(folder, dtype, trace, trace.most_held, tmp_path / "out")
    worst, where = compare(trace, result, reference, key=lambda rid: rid.split(":")[1])
    assert worst < TOL[torch.float32 if dtype == "float32" else torch.bfloat16], where


def test_command_line(models, tmp_path):
    """The generation command line on a Bofusun folder, and on a bare config.json with random weights
    (which also draws the distance table with its default length)."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    folder, cfg, _, _, _ = models["P"]
    common = ["--max-new-tokens", "7", "--max-len", "96", "--max-batch", "2"]
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--model", str(folder),
                           "--num-prompts", "3", "--prompt-len", "21", "--prompt", "hello", *common],
                          cwd=str(root), capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "4 requests, 2 rows" in proc.stdout and "> hello" in proc.stdout
    path = tmp_path / "config.json"
    path.write_text(json.dumps(TINY["R"][0]))
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--random-config", str(path),
                           "--num-prompts", "2", "--prompt-len", "30", "--dtype", "float32", *common],
                          cwd=str(root), capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "2 requests, 2 rows" in proc.stdout and "tok/s" in proc.stdout.splitlines()[-1]
