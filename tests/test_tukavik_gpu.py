"""Tukavik on the device: every mechanism's kernel alone against the plain implementation's
function, then whole models through the engine's step function in every cut (whole prompts, last
tokens one by one, portions down to two tokens, mixed batches with pages and state slots used
again, long decoding, first tokens), models whose weights make a lost key or a lost state show,
and greedy generation through the scheduler."""
import numpy as np
import pytest
import torch

import plain_tukavik as P
import traces
from tukavik_models import PAGE, TUK, make_dir, make_sharp_dir

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# errors are measured against the size of the logits (their standard deviation over the whole run)
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
STORE = {"float32": "float32", "bfloat16": "bfloat16"}
LENGTHS = {"A": [1, 2, 3, 17, 64, 130, 301], "B": [5, 129, 257, 16, 700], "C": [1, 9, 40, 63, 150]}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------- mechanisms
@pytest.mark.parametrize("width", [7, 64, 50])
def test_sinusoidal_embedding(width):
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    V = 23
    table = rng.standard_normal((V, width)).astype(np.float32)
    pos = [0, 1, 2, 15, 16, 17, 1000, 4095, 4096, 50000]
    tok = [int(t) for t in rng.integers(0, V, len(pos))]
    inv = torch.tensor(10000.0 ** (-2.0 * np.arange((width + 1) // 2) / width), dtype=torch.float64, device=DEV)
    out = torch.empty((len(pos), width), dtype=torch.float32, device=DEV)
    ops.embed(i32(tok), dev(table), out, positions=i32(pos), inv_freq=inv)
    want = np.stack([table[t] + P.sinusoid(1, width, first=p)[0] for t, p in zip(tok, pos)])
    assert np.abs(out.cpu().numpy() - want).max() < 1e-6


@pytest.mark.parametrize("form", ["layer", "rms"])
@pytest.mark.parametrize("width", [9, 20, 192, 1000])
def test_row_norms(form, width):
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    n, eps = 13, 1e-5
    x = rng.standard_normal((n, width + 5)) * 3 + 1.5
    g = rng.standard_normal(width) + 1
    fn = P.layer_norm if form == "layer" else P.rms_norm
    want = fn(x[:, 2:2 + width], g, eps)
    src = dev(x)[:, 2:2 + width]                     # a column range: a free row stride
    out = torch.empty((n, width), dtype=torch.float32, device=DEV)
    ops.norm_rows(src, dev(g), None, eps, out, form=form)
    assert np.abs(out.cpu().numpy() - want).max() < 2e-6
    # summed into a 32-bit stream
    res0 = rng.standard_normal((n, width))
    res = dev(res0)
    ops.norm_rows(src, dev(g), None, eps, res, form=form, add=True)
    assert np.abs(res.cpu().numpy() - (res0 + want)).max() < 3e-6
    # scattered into rows of a larger table, gathered from chosen rows, bfloat16 in and out
    rows = [5, 0, 17, 3, 40, 41, 39, 8, 9, 10, 2, 30, 31]
    table = torch.zeros((42, width), dtype=torch.bfloat16, device=DEV)
    xb = dev(x, torch.bfloat16)
    ops.norm_rows(xb[:, 2:2 + width], dev(g), None, eps, table, form=form, dst_rows=i32(rows))
    want_b = fn(xb[:, 2:2 + width].float().cpu().numpy().astype(np.float64), g, eps)
    got = table.float().cpu().numpy()
    assert np.abs(got[rows] - want_b).max() < 0.04 and np.abs(got[[1, 4, 6, 7]]).max() == 0
    pick = [12, 0, 7]
    out3 = torch.empty((3, width), dtype=torch.float32, device=DEV)
    ops.norm_rows(dev(x)[:, :width].contiguous(), None, None, eps, out3, form=form, src_rows=i32(pick))
    assert np.abs(out3.cpu().numpy() - fn(x[pick, :width], 1.0, eps)).max() < 2e-6


def test_xielu_and_depth_mix():
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(5)
    z = np.concatenate([rng.standard_normal(1000) * 3, [0.0, 1e-6, -1e-6, 20.0, -30.0]]).reshape(15, 67)
    p, q = 0.3, -0.7
    out = torch.empty((15, 67), dtype=torch.float32, device=DEV)
    ops.xielu(dev(z), out, float(P.softplus(p)), 0.5 + float(P.softplus(q)))
    want = P.xielu(z, p, q)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5 * max(1.0, np.abs(want).max())
    for T, E in ((3, 7), (5, 64)):                   # 21 elements: no vector load fits; 320: all do
        L = 4
        hist = torch.full((L + 1, T, E), 7.0, dtype=torch.float32, device=DEV)
        streams = [rng.standard_normal((T, E))]
        x = dev(streams[0])
        ops.depth_mix(x, hist, 1, None)
        assert torch.equal(x.cpu(), dev(streams[0]).cpu())
        for i in range(L):
            w = rng.standard_normal(i + 2)
            new = rng.standard_normal((T, E))
            streams.append(new)
            x = dev(new)
            ops.depth_mix(x, hist, i + 2, dev(w))
            assert np.abs(x.cpu().numpy() - P.depth_average(streams, w)).max() < 1e-5
            assert np.abs(hist[i + 1].cpu().numpy() - new).max() < 1e-6


@pytest.mark.parametrize("width", [10, 192, 600])
def test_sublayer_tail_in_one_launch_has_the_bits_of_its_three_kernels(width):
    """x += norm(y) g; the depth mix; the next norm: fused, against the plain functions and, bit
    for bit, against the separate kernels."""
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    T, eps, n_terms = 7, 1e-5, 4
    y, x0 = rng.standard_normal((T, width)) * 2, rng.standard_normal((T, width))
    g1, g2, w = rng.standard_normal(width) + 1, rng.standard_normal(width) + 1, rng.standard_normal(n_terms)
    old = [rng.standard_normal((T, width)) for _ in range(n_terms - 1)]
    summed = x0 + P.layer_norm(y, g1, eps)
    mixed = P.depth_average(old + [summed], w)
    for with_mix in (False, True):
        for out_dtype in (None, torch.float32, torch.bfloat16):
            hist = torch.zeros((n_terms + 1, T, width), dtype=torch.float32, device=DEV)
            hist[:n_terms - 1] = dev(np.stack(old))
            hist2 = hist.clone()
            x, x2 = dev(x0), dev(x0)
            h = torch.empty((T, width), dtype=out_dtype, device=DEV) if out_dtype else None
            ops.norm_add_tail(dev(y), dev(g1), eps, x, mix=(hist, n_terms, dev(w)) if with_mix else None,
                              then=(dev(g2), eps, "layer", h) if h is not None else None)
            want_x = mixed if with_mix else summed
            assert np.abs(x.cpu().numpy() - want_x).max() < 1e-5
            ops.norm_rows(dev(y), dev(g1), None, eps, x2, add=True)
            if with_mix:
                ops.depth_mix(x2, hist2, n_terms, dev(w))
                assert torch.equal(hist, hist2)
            assert torch.equal(x, x2)
            if h is not None:
                h2 = torch.empty_like(h)
                ops.norm_rows(x2, dev(g2), None, eps, h2)
                assert torch.equal(h, h2)
                assert np.abs(h.float().cpu().numpy() - P.layer_norm(want_x, g2, eps)).max() < (1e-5 if out_dtype == torch.float32 else 0.06)


def _scan_inputs(rng, n, W, gate_shift):
    """Projection weights that are identities, so that the plain function's gate, candidate and
    output-gate inputs are the rows themselves (plus a bias)."""
    h = rng.standard_normal((n, W)) * 2
    eye = np.eye(W)
    bz, bx = rng.standard_normal(W) * 0.3 + gate_shift, rng.standard_normal(W)
    return h, eye, bz, bx


@pytest.mark.parametrize("W", [150, 160])          # one channel a thread; four (16-byte loads)
@pytest.mark.parametrize("gate_shift", [0.0, -4.0])
def test_mingru_scan_short_and_chunked_with_carried_state(gate_shift, W):
    """Requests of unequal lengths in one step (single tokens beside portions longer than a chunk,
    chunk edges at 127/128/129), then the same sequences continued in a second step from the
    state the first left, with the slots in another order.  gate_shift -4 makes the gate open to
    about 2 %: the state then remembers hundreds of tokens, and one reset would show."""
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(11)
    for first, second in (([1, 5, 128, 64], [1, 1, 1, 1]),               # the one-launch way, then decoding
                          ([127, 1, 300, 129], [2, 256, 129, 1]),        # the chunked way both times
                          ([128, 385], [3, 2])):
        R = len(first)
        seqs = [_scan_inputs(rng, a + b, W, gate_shift) for a, b in zip(first, second)]
        want = [P.min_gru(h, eye, bz, eye, bx, eye, eye)[0] for h, eye, bz, bx in seqs]
        state = torch.zeros((R + 2, W), dtype=torch.float32, device=DEV)
        slots = list(rng.permutation(R + 2)[:R])
        done = [0] * R
        for lens in (first, second):
            rows = [np.concatenate([h[d:d + n] + bz, h[d:d + n] + bx, h[d:d + n]], 1)
                    for (h, _, bz, bx), d, n in zip(seqs, done, lens)]
            pre = dev(np.concatenate(rows))
            T = pre.shape[0]
            q_start = i32(np.concatenate([[0], np.cumsum(lens)]).tolist())
            y = torch.empty((T, W), dtype=torch.float32, device=DEV)
            need = ops.mingru_scan_workspace(R, W, T, max(lens))
            assert (need > 0) == (max(lens) > ops.GATED_SCAN_CHUNK)
            ws = torch.empty(max(need, 1), dtype=torch.float32, device=DEV)
            ops.mingru_scan(pre[:, :W], pre[:, W:2 * W], pre[:, 2 * W:], y, state, q_start, i32(slots), R, max(lens),
                            workspace=ws)
            got = y.cpu().numpy()
            t0 = 0
            for r, n in enumerate(lens):
                ref = want[r][done[r]:done[r] + n]
                assert np.abs(got[t0:t0 + n] - ref).max() < 2e-5 * max(1.0, np.abs(ref).max()), (lens, r)
                t0 += n
                done[r] += n
        free = [s for s in range(R + 2) if s not in slots]
        assert float(state[free].abs().max()) == 0.0         # nobody else's slot was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,heads,page", [(20, 3, 8), (64, 4, 16), (128, 2, 16), (9, 1, 4)])
def test_attention_over_shared_rows_far_keys_and_page_borders(dtype, rank, heads, page):
    """Attention where one cached row per position is key and value.  One key far back, one at a
    page's last place, one at a page's first are made to stand out in turn (the query points at
    it, twenty times longer): the result must be that row.  Random queries against the plain
    function; prompt portions and single tokens; pages in a scrambled order."""
    from sglang_c_b200.engine.runtime import Runtime
    from sglang_c_b200.csrc import ops
    rng = np.random.default_rng(rank)
    n = 333
    n_pages = (n + page - 1) // page + 3
    c = rng.standard_normal((n, rank))
    c /= np.linalg.norm(c, axis=1, keepdims=True)
    table = [int(p) for p in rng.permutation(n_pages)[:(n + page - 1) // page]]
    cache = torch.zeros((n_pages, 1, 1, page, rank), dtype=dtype, device=DEV)
    flat = cache.view(-1, rank)
    slot = [table[p // page] * page + p % page for p in range(n)]
    flat[torch.tensor(slot, device=DEV)] = dev(c, dtype)
    cq = flat[torch.tensor(slot, device=DEV)].float().cpu().numpy().astype(np.float64)      # as cached
    eye = np.concatenate([np.eye(rank)] * heads)
    bt = i32([table + [0] * 3])
    tol = 2e-5 if dtype == torch.float32 else 2e-2

    def run(q, positions, max_q_len, kernel="general"):
        T = len(positions)
        out = torch.empty((T, heads * rank), dtype=dtype, device=DEV)
        if kernel == "general":
            ops.attention_simt(dev(q, dtype), cache, bt, i32([0] * T), i32(positions), out, heads, 1.0, None,
                               max(positions) + 1, max_q_len=max_q_len, kv_shared=True)
        elif kernel == "decode":
            ops.attention_decode_shared(dev(q, dtype), cache, bt, i32([0] * T), i32(positions), out, heads, 1.0, None,
                                        max(positions) + 1)
        elif kernel.startswith("latent"):           # all heads a block; key ranges: as chosen, one, three, sixteen
            ops.attention_latent_decode(dev(q, dtype), cache, bt, i32([0] * T), i32(positions), out, heads, 1.0, None,
                                        max(positions) + 1, n_splits={"latent": None, "latent1": 1, "latent3": 3,
                                                                      "latent16": 16}[kernel])
        else:
            ops.attention_prefill_tc(dev(q, dtype), cache, bt, i32([0, T]), i32([positions[-1] + 1]), out, heads, 1.0,
                                     None, 1, T, kv_shared=True)
        return out.float().cpu().numpy()

    kernels = ["general"]
    if dtype == torch.bfloat16 and rank % 8 == 0:
        kernels += ["decode", "latent", "latent1", "latent3", "latent16"]
        assert ops.attention_latent_decode_supported(dev(np.zeros((1, heads * rank)), dtype), cache, heads)
    portion_kernels = ["general"] + (["tensor"] if dtype == torch.bfloat16 and rank in (64, 128) else [])
    # random queries: a portion of the last 70 positions, a portion that starts at 0, and single tokens
    q = rng.standard_normal((n, heads * rank)) * 1.5
    qr = dev(q, dtype).float().cpu().numpy().astype(np.float64)
    want = P.latent_attention(qr, cq, eye, eye, np.eye(heads * rank), heads, 1.0)
    for kernel in portion_kernels:
        got = run(q[n - 70:], list(range(n - 70, n)), 70, kernel)
        assert np.abs(got - want[n - 70:]).max() < tol, kernel
        got = run(q[:200], list(range(200)), 200, kernel)
        assert np.abs(got - want[:200]).max() < tol, kernel
    for kernel in kernels:
        for p in (0, 1, page - 1, page, 2 * page + 1, n - 1):
            assert np.abs(run(q[p:p + 1], [p], 1, kernel) - want[p:p + 1]).max() < tol, (kernel, p)
    # keys made to stand out
    for far in (0, 3, page - 1, page, 5 * page - 1, 5 * page, n - 2, n - 1):
        qf = np.tile(cq[far] * 40.0, heads)[None, :]
        for kernel in kernels:
            got = run(qf, [n - 1], 1, kernel)
            assert np.abs(got - np.tile(cq[far], heads)).max() < 5e-2, (kernel, far)
            if far > 0:       # and just out of sight: the query sits one place before it
                got = run(qf, [far - 1], 1, kernel)
                ref = P.latent_attention(np.repeat(qf, far, 0), cq[:far], eye, eye, np.eye(heads * rank), heads, 1.0)[-1]
                assert np.abs(got - ref).max() < max(tol, 2e-2 if dtype == torch.bfloat16 else 1e-4), (kernel, far)
        for kernel in portion_kernels[1:]:
            # the last query of a portion points at the far key; the one before it must not see position n-1
            qs = np.concatenate([q[n - 40:n - 1], qf])
            got = run(qs, list(range(n - 40, n)), 40, kernel)
            assert np.abs(got[-1] - np.tile(cq[far], heads)).max() < 5e-2, (kernel, far)
            assert np.abs(got[:-1] - want[n - 40:n - 1]).max() < tol, (kernel, far)


# ---------------------------------------------------------------------------- whole models
def requests_for(name):
    V = TUK[name]["vocab"]
    return {f"r{i}": traces.random_tokens(7 * i + ord(name), n, V) for i, n in enumerate(LENGTHS[name])}


_ref = {}


def reference(model_dir, requests):
    out = {}
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks))
        if key not in _ref:
            _ref[key] = P.forward_dir(model_dir, toks)
        out[rid] = _ref[key]
    return out


def relative_error(got, ref):
    err, where = traces.max_error(got, ref)
    size = float(np.concatenate([r.ravel() for r in ref.values()]).std())
    return err / size, where


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
    return traces.collect(steps, out, TUK[name]["vocab"]), eng


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("tukavik")
    return lambda name, store="float32", sharp=False: (make_sharp_dir if sharp else make_dir)(base, name, store)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions"])
def test_each_request_alone(dirs, tmp_path, name, dtype, mode):
    d = dirs(name, STORE[dtype])
    reqs = requests_for(name)
    steps = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions}[mode](reqs)
    got, _ = run_trace(d, dtype, name, steps, tmp_path)
    err, where = relative_error(got, reference(d, reqs))
    assert err < TOL[dtype], f"{mode}: error {err} of the logits' size at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(dirs, tmp_path, name, dtype):
    d = dirs(name, STORE[dtype])
    V = TUK[name]["vocab"]
    lens = [37, 64, 190, 21, 128, 55, 270, 33, 131, 48]
    reqs = {f"m{i}": traces.random_tokens(2000 + i, n, V) for i, n in enumerate(lens)}
    prompt_len = {rid: max(1, len(t) - 20 - 3 * i) for i, (rid, t) in enumerate(reqs.items())}
    steps = traces.mixed(reqs, prompt_len, seed=5, max_live=3, sizes=(5, 2, 11, 3, 140, 2, 8))
    peak = traces.peak_tokens(steps)
    assert peak < sum((n + 63) // 64 * 64 for n in lens)
    got, eng = run_trace(d, dtype, name, steps, tmp_path, max_tokens=peak, max_requests=3)
    err, where = relative_error(got, reference(d, reqs))
    assert err < TOL[dtype], f"mixed: error {err} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_sharp_model_in_every_cut(dirs, tmp_path, name, dtype):
    """Keys that carry weight and states that remember: first what the change does to the plain
    logits (a token changed far back must move the last logits), then every cut."""
    d = dirs(name, STORE[dtype], sharp=True)
    V = TUK[name]["vocab"]
    reqs = {f"s{i}": traces.random_tokens(900 + i, n, V) for i, n in enumerate([260, 45, 131])}
    ref = reference(d, reqs)
    toks = list(reqs["s0"])
    toks[3] = (toks[3] + 1) % V
    moved = np.abs(P.forward_dir(d, toks)[-1] - ref["s0"][-1]).max()
    size = float(ref["s0"].std())
    # (the 32-bit runs are the sharp ones: 20 times their bound; bfloat16's rounding is as large as
    # the move, there the kernels' own tests with a key made to stand out do the catching)
    assert moved > 20 * TOL["float32"] * size, moved / size
    prompt_len = {"s0": 200, "s1": 20, "s2": 129}
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs, 40), traces.portions(reqs, sizes=(2, 127, 3, 2, 64, 129)),
                  traces.mixed(reqs, prompt_len, seed=2, sizes=(130, 2, 16, 3))):
        got, _ = run_trace(d, dtype, name, steps, tmp_path)
        err, where = relative_error(got, ref)
        assert err < 3 * TOL[dtype], f"sharp: error {err} at {where}"


def test_mixed_results_do_not_depend_on_the_batch_in_32_bit(dirs, tmp_path):
    """In the 32-bit path a request's logits are the same in a mixed batch as alone, up to the
    rounding of the recurrence's chunked way (which a long portion takes and single tokens do not)."""
    d = dirs("A")
    V = TUK["A"]["vocab"]
    reqs = {f"q{i}": traces.random_tokens(500 + i, n, V) for i, n in enumerate([90, 33, 140, 7])}
    prompt_len = {rid: len(t) - 5 for rid, t in reqs.items()}
    mixed, _ = run_trace(d, "float32", "A", traces.mixed(reqs, prompt_len, seed=9), tmp_path)
    alone, _ = run_trace(d, "float32", "A", traces.whole(reqs), tmp_path)
    for rid in reqs:
        for p in alone[rid]:
            assert np.abs(mixed[rid][p] - alone[rid][p]).max() < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs(dirs, tmp_path, dtype):
    d = dirs("B", STORE[dtype])
    V = TUK["B"]["vocab"]
    reqs = {"long": traces.random_tokens(31, 420, V), "other": traces.random_tokens(32, 300, V)}
    steps = []
    for s in range(300):
        entries = []
        for rid, first in (("long", 120), ("other", 1)):
            if s == 0:
                entries.append({"id": rid, "tokens": reqs[rid][:first], "want": list(range(first))})
            elif first + s <= len(reqs[rid]):
                entries.append({"id": rid, "tokens": [reqs[rid][first + s - 1]], "want": [0]})
        steps.append({"step": s, "entries": entries, "end": []})
    steps[-1]["end"] = ["long", "other"]
    got, eng = run_trace(d, dtype, "B", steps, tmp_path, max_tokens=1024)
    ref = {"long": P.forward_dir(d, reqs["long"][:419]), "other": P.forward_dir(d, reqs["other"])}
    err, where = relative_error(got, ref)
    assert err < TOL[dtype], f"long decoding: error {err} at {where}"
    assert eng.graph_replays > 200, "steady decoding did not replay captured graphs"


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
    V = TUK[name]["vocab"]
    prompts = [traces.random_tokens(70 + i, n, V) for i, n in enumerate([5, 40, 1, 63, 100, 17])]
    s = sched_new(d, dtype=dtype, page_size=PAGE[name], max_tokens=384, max_requests=3, max_step_tokens=64,
                  prefill_chunk=24)
    got = generate(s, prompts, SamplingParams(temperature=0.0), max_new=12)
    for p, g in zip(prompts, got):
        assert len(g) == 12
        check_greedy(d, p, g, 1e-4 if dtype == "float32" else 5e-2)
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
    cfg.write_text(json.dumps(TUK["C"]))
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
