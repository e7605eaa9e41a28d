"""Buborax on the device: every mechanism's kernel alone against the plain implementation's
function, then whole models through the engine's step function in every cut (whole prompts, last
tokens one by one, portions down to two tokens, mixed batches with pages and state slots used
again, long decoding), models whose constants make a lost key, a window edge or a lost state show,
and greedy generation through the scheduler and the command line."""
import numpy as np
import pytest
import torch

import plain_buborax as P
import traces
from buborax_models import BUB, PAGE, make_dir, make_sharp_dir

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# Errors are measured against the size of the logits (their standard deviation over the whole run).
# The 32-bit bound holds at every position and is the sharp one: edges and states are pinned by it
# (noise of half a unit in the last place of the 32-bit weights moves the plain implementation's
# logits by up to 5e-5 of their size in these models, a lost key or state by a hundred times that).
# In bfloat16 these narrow random models are noisy (a head's read-out that happens to be small is
# normed up with its rounding), so there the bound is on the bulk of the positions: a key, a state
# or a page that is lost moves most positions by the logits' own size.
TOL = {"float32": 2e-4, "bfloat16": 0.12}
BF16_MEDIAN, BF16_SHARE_OVER, BF16_WORST = 0.05, 0.08, 1.5
STORE = {"float32": "float32", "bfloat16": "bfloat16"}
LENGTHS = {"A": [1, 2, 3, 17, 49, 130, 211], "B": [5, 129, 257, 16, 301], "C": [1, 9, 40, 63, 150]}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def f64(t):
    return t.float().cpu().numpy().astype(np.float64)


# ---------------------------------------------------------------------------- mechanisms
@pytest.mark.parametrize("E,groups", [(64, 2), (50, 5), (128, 1), (36, 9), (192, 3), (7, 7)])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_rms_norm_in_groups(E, groups, out):
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(E + groups)
    x = rng.standard_normal((11, E)) * np.linspace(0.01, 30.0, E)      # parts of very different sizes
    gain = 1.0 + 0.3 * rng.standard_normal(E)
    want = P.group_norm(x, gain, 1e-5, groups)
    y = torch.zeros((11, E), dtype=out, device=DEV)
    ops.norm_rows(dev(x), dev(gain), None, 1e-5, y, form="rms", groups=groups)
    assert np.abs(f64(y) - want).max() < (1e-5 if out == torch.float32 else 2e-2) * np.abs(want).max()
    if groups > 1:                    # (and the groups are not the whole row's statistics)
        assert np.abs(P.group_norm(x, gain, 1e-5, 1) - want).max() > 0.1


@pytest.mark.parametrize("F,dtype", [(33, torch.float32), (64, torch.bfloat16), (40, torch.bfloat16)])
def test_gelu_gate_with_a_multiplier(F, dtype):
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(F)
    gu = torch.tensor(rng.standard_normal((9, 2 * F)) * 2.5, dtype=dtype, device=DEV)
    z = torch.zeros((9, F), dtype=dtype, device=DEV)
    ops.gated_act(gu, z, act="gelu_tanh", mult=0.7)
    g = f64(gu)
    want = P.gelu_tanh(g[:, :F]) * g[:, F:] * 0.7
    assert np.abs(f64(z) - want).max() < (2e-6 if dtype == torch.float32 else 1e-2) * np.abs(want).max()
    assert np.abs(P.silu(g[:, :F]) * g[:, F:] * 0.7 - want).max() > 0.05        # not the other activation


def test_norm_of_each_head_without_a_gate():
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(5)
    H, V = 3, 10
    o = rng.standard_normal((7, H, V)) * np.array([0.01, 1.0, 50.0])[None, :, None]
    gain = 1.0 + 0.2 * rng.standard_normal(V)
    y = torch.zeros((7, H * V), device=DEV)
    ops.gated_norm(dev(o.reshape(7, H * V)), None, dev(gain), y, H, V, 1e-5, "none")
    assert np.abs(f64(y) - P.rms_norm(o, gain, 1e-5).reshape(7, H * V)).max() < 1e-5


@pytest.mark.parametrize("H,D,V", [(4, 16, 24), (2, 64, 80), (3, 7, 5), (1, 200, 33), (2, 128, 1), (1, 48, 32)])
def test_row_gated_state_in_portions(H, D, V):
    """Three requests of unequal lengths in shuffled slots, whole and cut into portions (the state is
    carried through its slot), with lower bounds close to one so that the first tokens still count."""
    from sglang_c_b200.csrc import ops
    _row_gated_in_portions(ops, H, D, V)


def _row_gated_in_portions(ops, H, D, V):
    rng = np.random.default_rng(H * 1000 + D)
    lens = [45, 1, 18]
    lower = 0.97 + 0.029 * rng.random(H * D)
    data, want = [], []
    for n in lens:
        qx, fx, v = rng.standard_normal((n, H * D)), rng.standard_normal((n, H * D)), rng.standard_normal((n, H * V))
        f = lower + (1.0 - lower) * P.sigmoid(fx)
        data.append((qx, fx, v))
        want.append(P.row_gated_state(P.silu(qx).reshape(n, H, D), f.reshape(n, H, D), v.reshape(n, H, V)))
    qx, fx, v = data[0]
    f = (lower + (1.0 - lower) * P.sigmoid(fx)).reshape(-1, H, D)
    short = P.row_gated_state(P.silu(qx[1:]).reshape(-1, H, D), f[1:], v[1:].reshape(-1, H, V))[0]
    assert np.abs(short[-1] - want[0][0][-1]).max() > 1e-3              # the first token shows at the end
    for cuts in ([[45, 1, 18]], [[9, 1, 2], [2, 0, 16], [34, 0, 0]]):
        state = torch.zeros((6, H, D, V), device=DEV)
        state[[0, 1, 3]] = 7.0                      # other slots' contents must neither be read nor touched
        slots = [4, 2, 5]
        done = [0, 0, 0]
        got = [np.zeros((n, H * V)) for n in lens]
        for cut in cuts:
            live = [r for r in range(3) if cut[r] > 0]
            rows = [np.concatenate([data[r][j][done[r]:done[r] + cut[r]] for r in live]) for j in range(3)]
            T = sum(cut)
            out = torch.zeros((T, H * V), device=DEV)
            q_start = np.concatenate([[0], np.cumsum([cut[r] for r in live])])
            ops.matrix_state("row_gate", dev(rows[0]), dev(rows[1]), dev(rows[2]), out, state, i32(q_start),
                             i32([slots[r] for r in live]), len(live), H, H, D, V, silu_in=True, lower=dev(lower))
            o = f64(out)
            for j, r in enumerate(live):
                got[r][done[r]:done[r] + cut[r]] = o[q_start[j]:q_start[j + 1]]
                done[r] += cut[r]
        for r in range(3):
            assert np.abs(got[r] - want[r][0].reshape(lens[r], H * V)).max() < 2e-4 * max(1.0, np.abs(want[r][0]).max())
            assert np.abs(f64(state[slots[r]]) - want[r][1]).max() < 1e-4
        assert float((state[[0, 1, 3]] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("H,R,Rd,dims", [(3, 40, 8, 6), (2, 96, 32, 32), (1, 13, 6, 4), (4, 16, 2, 2)])
def test_latent_row_and_queries_are_normed_and_turned(H, R, Rd, dims):
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(R)
    T, W, base = 9, R + Rd, 500.0
    pos = np.array([0, 1, 2, 70, 71, 1000, 4095, 4096, 30000])
    qx, low = rng.standard_normal((T, H, W)), rng.standard_normal((T, W)) * 3
    gain = 1.0 + 0.2 * rng.standard_normal(R)
    want_q = qx.copy()
    want_q[..., R:] = P.rotate_pairs(qx[..., R:], pos.astype(np.float64), dims, base)
    want_row = np.concatenate([P.rms_norm(low[:, :R], gain, 1e-5),
                               P.rotate_pairs(low[:, R:], pos.astype(np.float64), dims, base)], 1)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64, device=DEV)
    slots = [17, 3, 4, 0, 9, 11, 2, 5, 8]
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        q = torch.zeros((T, H * W), dtype=dt, device=DEV)
        rows = torch.zeros((20, W), dtype=dt, device=DEV)
        ops.latent_rope(dev(qx.reshape(T, H * W)), dev(low), dev(gain), 1e-5, i32(pos), freq, 1.0, dims, "neighbours",
                        q, rows, i32(slots), H, R, Rd)
        assert np.abs(f64(q).reshape(T, H, W) - want_q).max() < tol * np.abs(want_q).max()
        assert np.abs(f64(rows)[slots] - want_row).max() < tol * np.abs(want_row).max()
        untouched = [s for s in range(20) if s not in slots]
        assert float(rows[untouched].abs().max()) == 0.0
    # the other pairing is another function
    halves = torch.zeros((T, H * W), device=DEV)
    ops.latent_rope(dev(qx.reshape(T, H * W)), None, None, 1e-5, i32(pos), freq, 1.0, dims, "halves", halves, None, None,
                    H, R, Rd)
    if dims > 2:
        assert np.abs(f64(halves).reshape(T, H, W) - want_q).max() > 1e-2


def _bf16(a):
    """The values rounded to what bfloat16 holds (so that a bfloat16 cache keeps them exactly)."""
    return torch.tensor(a, dtype=torch.float32).to(torch.bfloat16).double().numpy()


def _talk_case(rng, n, H, G, D, far=()):
    """Projected queries, keys and gates of n tokens; for (i, j) of `far` the key at j is made to
    stand out for the query at i (both unit-normed alike, the key as projected 40 times as long: as
    a value it then dominates whatever sees it)."""
    q, k = rng.standard_normal((n, H, D)), rng.standard_normal((n, G, D))
    for i, j in far:
        k[j] = 40.0 * q[i, ::H // G] / np.sqrt((q[i, ::H // G] ** 2).mean(-1, keepdims=True))
    return q, _bf16(k), rng.standard_normal((n, H * D))


@pytest.mark.parametrize("H,G,D,window,page", [(4, 2, 16, 37, 16), (2, 1, 32, None, 16), (3, 3, 10, 8, 8),
                                              (4, 4, 64, 130, 16), (1, 1, 7, 3, 8), (6, 2, 24, 300, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_talking_heads_attention_windows_far_keys_and_portions(H, G, D, window, page, dtype):
    _talk_in_cuts(H, G, D, window, page, dtype, tiled=False)


@pytest.mark.parametrize("H,G,D,window,page", [(4, 2, 32, 37, 16), (2, 1, 64, None, 16), (3, 3, 48, 8, 8),
                                              (8, 2, 128, 130, 32), (1, 1, 32, 3, 8), (6, 2, 96, 300, 16),
                                              (16, 4, 32, 33, 16), (5, 5, 64, 32, 24), (2, 2, 64, 16, 16)])
@pytest.mark.parametrize("max_keys", [None, 1 << 20])
@pytest.mark.parametrize("split", [True, False])
def test_talking_heads_attention_in_tiles(H, G, D, window, page, max_keys, split):
    """max_keys None: the longest request's length, so that every key is staged once where that fits
    (and twice through two buffers where it does not); a bound far off: always through two buffers
    where there is no window.  split: small grids divide a tile's keys over a cluster of blocks (some
    of which get no keys where the window is short or the request has just begun); without it every
    tile of queries is one block's."""
    from sglang_c_b200.csrc import ops
    ops.set_kernel_choice(talk_key_split=split)
    try:
        _talk_in_cuts(H, G, D, window, page, torch.bfloat16, tiled=True, max_keys=max_keys)
    finally:
        ops.set_kernel_choice(talk_key_split=True)


def _talk_in_cuts(H, G, D, window, page, dtype, tiled, max_keys=None):
    """Two requests over shuffled pages, whole, then in portions with single tokens at the end.  In the
    first request the key just inside the window of the last query, the key just outside the window
    of the query before it (and, without a window, a key hundreds back) stand out: a window one token
    off, or a lost key, changes the result by its own size.  tiled: the tensor-core form, which
    takes the requests' first rows and lengths in place of a request and a position per token."""
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(H * 100 + D)
    lens = [333, 70]
    scale, mult = 6.0 / np.sqrt(D), 0.7
    last = lens[0] - 1
    w = window if window is not None else lens[0]
    far = [(last, max(last - w + 1, 3))] + ([(last - 1, last - 1 - w)] if window is not None else [])
    cases = [_talk_case(rng, lens[0], H, G, D, far), _talk_case(rng, lens[1], H, G, D)]
    gq, gk = 1.0 + 0.2 * rng.standard_normal(D), 1.0 + 0.2 * rng.standard_normal(D)
    talk = np.eye(H) * 0.8 + 0.3 * rng.standard_normal((H, H))
    plain = lambda c, size: P.talking_heads(c[0], c[1], gq, gk, talk, scale, size, 1e-6).reshape(len(c[0]), H * D)
    want = [plain(c, window) * P.sigmoid(c[2]) * mult for c in cases]
    if window is not None:             # the stand-out keys matter: one token off is another result
        assert np.abs(plain(cases[0], window + 1)[last - 1] - plain(cases[0], window)[last - 1]).max() > 1.0
        assert np.abs(plain(cases[0], window - 1)[last] - plain(cases[0], window)[last]).max() > 1.0
    n_pages = {16: 40, 8: 80}.get(page, 30)
    blocks = [(n + page - 1) // page for n in lens]
    perm = rng.permutation(n_pages)
    tables = np.zeros((2, max(blocks)), dtype=np.int64)
    tables[0, :blocks[0]], tables[1, :blocks[1]] = perm[:blocks[0]], perm[blocks[0]:blocks[0] + blocks[1]]
    xs = [np.concatenate([c[0].reshape(len(c[0]), -1), c[1].reshape(len(c[1]), -1)], 1) for c in cases]
    gates = [c[2] for c in cases]
    slopes = dev(P.head_slopes(H))
    tol = 2e-4 if dtype == torch.float32 else 1e-2
    tail = [[(lo, lo + 1), (lo - 263, lo - 262)] for lo in range(329, 333)]
    for cuts in ([[(0, 333), (0, 70)]], [[(0, 141), (0, 9)], [(141, 143), (9, 65)], [(143, 329), (65, 66)]] + tail):
        cache = torch.zeros((n_pages, 1, G, page, D), dtype=dtype, device=DEV)
        got = [np.zeros_like(x) for x in want]
        for step in cuts:
            live = [(r, lo, hi) for r, (lo, hi) in enumerate(step) if hi > lo]
            x = dev(np.concatenate([xs[r][lo:hi] for r, lo, hi in live]))
            gate = dev(np.concatenate([gates[r][lo:hi] for r, lo, hi in live]))
            pos = np.concatenate([np.arange(lo, hi) for _, lo, hi in live])
            slots = np.concatenate([tables[r][np.arange(lo, hi) // page] * page + np.arange(lo, hi) % page
                                    for r, lo, hi in live])
            token_req = np.concatenate([np.full(hi - lo, j) for j, (_, lo, hi) in enumerate(live)])
            bt = np.stack([tables[r] for r, _, _ in live])
            T = len(pos)
            qn = torch.zeros((T, H * D), device=DEV)
            ops.talk_prep(x, dev(gq), dev(gk), 1e-6, qn, cache, i32(slots), H, G, D, page)
            out = torch.zeros((T, H * D), dtype=dtype, device=DEV)
            if tiled:
                counts = [hi - lo for _, lo, hi in live]
                q_start = np.concatenate([[0], np.cumsum(counts)])
                assert ops.talk_attention_tiles(qn, cache, i32(bt), i32(q_start), i32([hi for _, _, hi in live]),
                                                slopes, dev(talk.reshape(-1)), gate, out, len(live), max(counts), H,
                                                G, D, page, scale, 1e-6, mult, window,
                                                max_keys=max_keys if max_keys else max(hi for _, _, hi in live))
            else:
                ops.talk_attention(qn, cache, i32(bt), i32(token_req), i32(pos), slopes, dev(talk.reshape(-1)), gate,
                                   out, H, G, D, page, scale, 1e-6, mult, window)
            o = f64(out)
            at = 0
            for r, lo, hi in live:
                got[r][lo:hi] = o[at:at + hi - lo]
                at += hi - lo
        for r in range(2):
            err = np.abs(got[r] - want[r]).max(-1) / np.maximum(np.abs(want[r]).max(-1), 1.0)
            assert err.max() < tol, (cuts[0], r, int(err.argmax()), float(err.max()))


def test_rows_cast_into_a_column_range():
    from sglang_c_b200.csrc import ops
    x = torch.randn((5, 12), device=DEV)
    for dt in (torch.float32, torch.bfloat16):
        rows = torch.full((5, 24), 9.0, dtype=dt, device=DEV)
        ops.cast_rows(x, rows[:, 12:])
        assert torch.equal(rows[:, 12:], x.to(dt)) and float((rows[:, :12] - 9.0).abs().max()) == 0.0


# ---------------------------------------------------------------------------- whole models
def requests_for(name):
    V = BUB[name]["vocab"]
    return {f"r{i}": traces.random_tokens(11 * i + ord(name), n, V) for i, n in enumerate(LENGTHS[name])}


def reference(model_dir, requests):
    return {rid: P.forward_dir(model_dir, toks) for rid, toks in requests.items()}


def relative_error(got, ref):
    err, where = traces.max_error(got, ref)
    size = float(np.concatenate([r.ravel() for r in ref.values()]).std())
    return err / size, where


def accept(got, ref, dtype, what, factor=1.0):
    """32-bit: every position within the bound.  bfloat16: the bulk of the positions (see TOL)."""
    err, where = relative_error(got, ref)
    if dtype == "float32":
        assert err < factor * TOL[dtype], f"{what}: error {err} of the logits' size at {where}"
        return
    size = float(np.concatenate([r.ravel() for r in ref.values()]).std())
    e = np.array([np.abs(got[rid][p].astype(np.float64) - r[p]).max() / size for rid, r in ref.items() for p in sorted(got[rid])])
    said = f"{what}: median {np.median(e):.3g}, share over {TOL[dtype]}: {np.mean(e > TOL[dtype]):.3g}, worst {err:.3g} at {where}"
    assert np.median(e) < BF16_MEDIAN and np.mean(e > TOL[dtype]) < BF16_SHARE_OVER and err < BF16_WORST, said


def run_trace(model_dir, dtype, name, steps, tmp_path, max_tokens=None, max_step_tokens=1024, max_requests=4):
    from sglang_c_b200.engine import Engine
    from sglang_c_b200.engine.replay import replay
    ps = PAGE[name]
    n_pages = (max_tokens or traces.peak_tokens(steps)) // ps
    eng = Engine.from_dir(model_dir, dtype=dtype, page_size=ps, n_pages=n_pages, max_requests=max_requests,
                          max_step_tokens=max_step_tokens)
    out = str(tmp_path / "out")
    done = []
    replay(eng, traces.to_lines(steps), out, emit=done.append)
    assert done == [f"done {st['step']}" for st in steps]
    eng.cache.check()
    assert eng.cache.n_free_pages() == n_pages and eng.cache.n_free_slots() == max_requests
    return traces.collect(steps, out, BUB[name]["vocab"]), eng


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("buborax")
    return lambda name, store="float32", sharp=False: (make_sharp_dir if sharp else make_dir)(base, name, store)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions"])
def test_each_request_alone(dirs, tmp_path, name, dtype, mode):
    d = dirs(name, STORE[dtype])
    reqs = requests_for(name)
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, 45), "portions": traces.portions}[mode](reqs)
    got, _ = run_trace(d, dtype, name, steps, tmp_path)
    accept(got, reference(d, reqs), dtype, mode)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(dirs, tmp_path, name, dtype):
    d = dirs(name, STORE[dtype])
    V = BUB[name]["vocab"]
    lens = [37, 64, 150, 21, 128, 55, 33, 131, 48]
    reqs = {f"m{i}": traces.random_tokens(2000 + i, n, V) for i, n in enumerate(lens)}
    prompt_len = {rid: max(1, len(t) - 20 - 3 * i) for i, (rid, t) in enumerate(reqs.items())}
    steps = traces.mixed(reqs, prompt_len, seed=5, max_live=3, sizes=(5, 2, 11, 3, 140, 2, 8))
    peak = traces.peak_tokens(steps)
    assert peak < sum((n + 63) // 64 * 64 for n in lens)
    got, eng = run_trace(d, dtype, name, steps, tmp_path, max_tokens=peak, max_requests=3)
    accept(got, reference(d, reqs), dtype, "mixed")


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sharp_model_in_every_cut(dirs, tmp_path, name, dtype="float32"):
    """Keys that carry weight and states that remember: first what the change does to the plain
    logits (a token changed far back must move the last logits), then every cut.  (32-bit only: with
    scores this large the rounding of bfloat16 queries and keys moves the logits as much as a lost key.)"""
    d = dirs(name, STORE[dtype], sharp=True)
    V = BUB[name]["vocab"]
    reqs = {f"s{i}": traces.random_tokens(900 + i, n, V) for i, n in enumerate([200, 45, 131])}
    ref = reference(d, reqs)
    toks = list(reqs["s0"])
    toks[3] = (toks[3] + 1) % V
    moved = np.abs(P.forward_dir(d, toks)[-1] - ref["s0"][-1]).max()
    size = float(ref["s0"].std())
    assert moved > 40 * TOL["float32"] * size, moved / size
    prompt_len = {"s0": 150, "s1": 20, "s2": 129}
    cuts = {"whole": traces.whole(reqs), "tail": traces.tail_decoded(reqs, 40),
            "portions": traces.portions(reqs, sizes=(2, 127, 3, 2, 64, 23)),
            "mixed": traces.mixed(reqs, prompt_len, seed=2, sizes=(130, 2, 16, 3))}
    errs = {}
    for cut, steps in cuts.items():
        got, _ = run_trace(d, dtype, name, steps, tmp_path)
        errs[cut] = relative_error(got, ref)
    assert all(e < 4 * TOL[dtype] for e, _ in errs.values()), f"sharp: {errs}"


def test_mixed_results_do_not_depend_on_the_batch_in_32_bit(dirs, tmp_path):
    """In the 32-bit path every row has one order of additions whatever else is in the step: a
    request's logits in a mixed batch are those of the request alone."""
    d = dirs("A")
    V = BUB["A"]["vocab"]
    reqs = {f"q{i}": traces.random_tokens(500 + i, n, V) for i, n in enumerate([90, 33, 140, 7])}
    prompt_len = {rid: len(t) - 5 for rid, t in reqs.items()}
    mixed, _ = run_trace(d, "float32", "A", traces.mixed(reqs, prompt_len, seed=9), tmp_path)
    alone, _ = run_trace(d, "float32", "A", traces.whole(reqs), tmp_path)
    for rid in reqs:
        for p in alone[rid]:
            assert np.abs(mixed[rid][p] - alone[rid][p]).max() < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs(dirs, tmp_path, dtype):
    """Two requests decoded for 240 steps: windows pass over decoded tokens, pages behind them return."""
    d = dirs("A", STORE[dtype])
    V = BUB["A"]["vocab"]
    reqs = {"long": traces.random_tokens(31, 300, V), "other": traces.random_tokens(32, 240, V)}
    steps = []
    for s in range(240):
        entries = []
        for rid, first in (("long", 60), ("other", 1)):
            if s == 0:
                entries.append({"id": rid, "tokens": reqs[rid][:first], "want": list(range(first))})
            elif first + s <= len(reqs[rid]):
                entries.append({"id": rid, "tokens": [reqs[rid][first + s - 1]], "want": [0]})
        steps.append({"step": s, "entries": entries, "end": []})
    steps[-1]["end"] = ["long", "other"]
    got, eng = run_trace(d, dtype, "A", steps, tmp_path, max_tokens=640)
    ref = {"long": P.forward_dir(d, reqs["long"][:299]), "other": P.forward_dir(d, reqs["other"])}
    accept(got, ref, dtype, "long decoding")
    assert eng.graph_replays > 150, "steady decoding did not replay captured graphs"


def check_greedy(model_dir, prompt, got, tie):
    cfg, w = P.read_model_dir(model_dir)
    seq = list(prompt)
    for t in got:
        lg = P.forward(cfg, w, seq)[-1]
        best = int(np.argmax(lg))
        assert t == best or lg[best] - lg[t] < tie * lg.std(), (t, best, float(lg[best] - lg[t]))
        seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(dirs, name, dtype):
    """The entry point a user calls: prompts of unequal lengths in one batch, prompt portions of 24
    tokens, few pages (so requests wait for pages and slots that others give back)."""
    from sglang_c_b200.engine import generate, sched_new
    from sglang_c_b200.sampling import SamplingParams
    d = dirs(name, STORE[dtype])
    V = BUB[name]["vocab"]
    prompts = [traces.random_tokens(70 + i, n, V) for i, n in enumerate([5, 40, 1, 63, 100, 17])]
    s = sched_new(d, dtype=dtype, page_size=PAGE[name], max_tokens=384, max_requests=3, max_step_tokens=64,
                  prefill_chunk=24)
    got = generate(s, prompts, SamplingParams(temperature=0.0), max_new=10)
    for p, g in zip(prompts, got):
        assert len(g) == 10
        # (bfloat16: a token whose logit lies within that precision's bound of the best one may win)
        check_greedy(d, p, g, 1e-4 if dtype == "float32" else TOL["bfloat16"])
    st = s.get_stats()
    assert st.n_finished == len(prompts) and st.pool_free == st.pool_pages


def test_command_line_generates_from_a_random_folder(tmp_path):
    """bin/sglc: a random folder written from a config.json, then greedy generation from it."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(BUB["C"]))
    d = str(tmp_path / "model")
    prompt = [5, 17, 3, 99, 42]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sglc"), "--random-weights", "11", "--config", str(cfg),
                           "--init", "varied", "--save-model", d, "--dtype", "float32", "--prompt",
                           " ".join(map(str, prompt)), "--max-new", "8", "--temperature", "0", "--page-size", "8"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ids = [int(t) for t in proc.stdout.strip().splitlines()[-1].split()]
    assert ids[:len(prompt)] == prompt and len(ids) == len(prompt) + 8
    check_greedy(d, prompt, ids[len(prompt):], 1e-4)
