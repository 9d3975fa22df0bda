"""Sosutar on the GPU: every mechanism's kernels against the plain implementation, then whole
models through the engine (prompts, token-by-token decoding, portions, unequal batches, slots and
pages used again, long decoding, graph replay) and greedy generation through the session."""
import math

import numpy as np
import pytest
import torch

import ember_cpp_b200 as E
from ember_cpp_b200.cache.sequence_cache import SequenceCache
from ember_cpp_b200.engine.plan import StepPlan, build_step
from ember_cpp_b200.parts import CacheNeed

import plain_sosutar as P
import sosutar_util as U
from conftest import run_batch

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
OP_TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


@pytest.fixture(scope="module")
def ops():
    from ember_cpp_b200.csrc.ops import CudaOps
    return CudaOps()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: U.write_model(str(tmp_path_factory.mktemp(name)), U.config(name), U.SEEDS[name]) for name in U.CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: P.PlainSosutar(folder) for name, folder in folders.items()}


def rnd(seed, *shape, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def f64(t):
    return t.detach().double().cpu().numpy()


def close(got, want, tol):
    got, want = f64(got) if torch.is_tensor(got) else got, np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= tol * max(np.abs(want).max(), 1e-9), np.abs(got - want).max() / np.abs(want).max()


def plan_of(seqs):
    """seqs: (slot, positions held, new tokens); a step's description without a cache."""
    host = build_step([(s, [0] * n, []) for s, _, n in seqs], {s: a for s, a, _ in seqs}, [], 1)
    return StepPlan(host, torch.from_numpy(host.packed).cuda())


STEPS = ([(3, 2), (1, 41), (4, 1)], [(3, 37), (1, 1), (4, 2)], [(1, 1), (-1, 1), (3, 1), (4, 1)], [(4, 5), (3, 7)], [(1, 1)])
LENGTHS = {3: 47, 1: 44, 4: 9}


def feed(step_fn, data, dt, stride):
    """Three sequences fed in unequal steps (prompts, portions, one token each, a padding sequence in between);
    step_fn(plan, rows of the step) -> rows of the step.  Returns the outputs per sequence."""
    got = {s: [] for s in LENGTHS}
    at = {s: 0 for s in LENGTHS}
    for step in STEPS:
        seqs = [(s, at.get(s, 0), n) for s, n in step]
        rows = torch.cat([data[s][at[s]:at[s] + n] if s >= 0 else torch.zeros(n, stride, dtype=dt) for s, _, n in seqs]).cuda()
        out = step_fn(plan_of(seqs), rows)
        row = 0
        for s, _, n in seqs:
            if s >= 0:
                got[s].append(out[row:row + n])
                at[s] += n
            else:
                assert not out[row:row + n].any()
            row += n
    return {s: torch.cat(v) for s, v in got.items()}


# ------------------------------------------------------------------------------ rows: norms of q, k and v, gates, sums of branches
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv, hd, vd, every", [(4, 2, 16, 32, 8), (3, 3, 12, 10, 1), (1, 1, 64, 64, 48)])
def test_norms_of_q_k_and_v_and_the_query_temperature(ops, dtype, heads, kv, hd, vd, every):
    T, eps, coef = 70, 1e-5, 0.7
    width = (heads + kv) * hd + kv * vd
    proj = rnd(1, T, width + 13, scale=2.0)                      # wider rows: the gate's columns lie behind
    qg, kg = rnd(2, heads * hd, scale=0.2) + 1, rnd(3, kv * hd, scale=0.2) + 1
    pos = torch.arange(57, 57 + T, dtype=torch.int32)
    x = f64(proj)
    q = P.rms_norm(x[:, :heads * hd], f64(qg), eps) * np.array([P.temperature(int(p), coef, every) for p in pos])[:, None]
    k = P.rms_norm(x[:, heads * hd:(heads + kv) * hd], f64(kg), eps)
    v = P.rms_unit(x[:, (heads + kv) * hd:width].reshape(T, kv, vd), eps).reshape(T, kv * vd)
    got = ops.qkv_norm(proj.cuda(), pos.cuda(), heads, kv, hd, vd, DT[dtype], q_gain=qg.cuda(), k_gain=kg.cuda(), unit_values=True,
                       eps=eps, temp_coef=coef, temp_every=every)
    close(got, np.concatenate([q, k, v], 1), OP_TOL[dtype])
    plain = ops.qkv_norm(proj.cuda(), pos.cuda(), heads, kv, hd, vd, DT[dtype])          # nothing asked for: the rows as they are
    close(plain, x[:, :width], OP_TOL[dtype])


def test_the_temperature_steps_exactly_where_the_floor_does(ops):
    pos = torch.tensor([0, 6, 7, 8, 14, 15, 16, 62, 63, 64], dtype=torch.int32)
    proj = torch.ones(len(pos), 3 * 8)
    got = f64(ops.qkv_norm(proj.cuda(), pos.cuda(), 1, 1, 8, 8, torch.float32, temp_coef=0.75, temp_every=8))[:, 0]
    want = [1 + 0.75 * math.log(k + 1) for k in (0, 0, 1, 1, 1, 2, 2, 7, 8, 8)]
    assert np.abs(got - want).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_on_rows(ops, dtype):
    a, proj = rnd(1, 19, 40).to(DT[dtype]), rnd(2, 19, 77, scale=2.0)
    for gate, fn in (("sigmoid", P.sigmoid), ("silu", P.silu)):
        close(ops.gate_mul(a.cuda(), proj.cuda(), 24, gate), f64(a) * fn(f64(proj[:, 24:64])), OP_TOL[dtype])


def test_branches_normed_one_by_one_are_summed_with_a_gain_in_one_launch(ops):
    rows, d, eps = 21, 136, 1e-5
    x, gain = rnd(1, rows, d), rnd(2, d, scale=0.3) + 1
    a, b, c = rnd(3, rows, d, scale=5.0).cuda(), rnd(4, rows, d, scale=0.01).cuda(), rnd(5, rows, d).cuda()
    wa, wb = rnd(6, d, scale=0.2) + 1, rnd(7, d, scale=0.2) + 1
    want = f64(x) + f64(gain) * (0.5 * P.rms_norm(f64(a), f64(wa), eps) + 0.5 * P.rms_norm(f64(b), f64(wb), eps) + 0.3 * f64(c))
    before = ops.launches
    got = ops.add_branches(x.clone().cuda(), [(a, 0.5, wa.cuda()), (b, 0.5, wb.cuda()), (c, 0.3)], gain.cuda(), eps)
    assert ops.launches == before + 1
    close(got, want, 3e-6)
    close(ops.add_branches(x.clone().cuda(), [(c, 1.0, None)], None, eps), f64(x) + f64(c), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M", [3, 40, 200, 700])
def test_squared_relu_in_a_product(ops, dtype, M):
    a, w = rnd(1, M, 64).to(DT[dtype]), rnd(2, 48, 64, scale=0.2).to(DT[dtype])
    got = ops.linear(a.cuda(), w.cuda(), None, act="relu2", out_dtype=DT[dtype])
    close(got, np.square(np.maximum(f64(a) @ f64(w).T, 0)), OP_TOL[dtype])


def test_the_embedding_scales_the_tokens_row_alone(ops):
    table, pos = rnd(1, 30, 24).bfloat16(), rnd(2, 50, 24).bfloat16()
    tokens, positions = torch.tensor([3, 29, 0], dtype=torch.int32), torch.tensor([7, 0, 49], dtype=torch.int32)
    got = ops.embed(tokens.cuda(), positions.cuda(), table.cuda(), pos.cuda(), token_scale=16.0)
    close(got, f64(table)[tokens.long()] * 16.0 + f64(pos)[positions.long()], 1e-6)


# ------------------------------------------------------------------------------ mLSTM
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, dim, vdim, cap", [(2, 16, 24, 6.0), (1, 12, 10, 30.0), (3, 48, 56, 12.0), (2, 80, 200, 3.0), (1, 130, 8, 15.0)])
def test_mlstm_gates_recurrence_and_head_norm_over_steps(ops, dtype, heads, dim, vdim, cap):
    """Against the plain recurrence on the whole sequences.  The state rows start as NaN: a sequence that begins
    must not read them."""
    dt, width, eps = DT[dtype], 72, 1e-5
    qk, inner = heads * dim, heads * vdim
    stride = -(-(2 * qk + 2 * inner) // 8) * 8
    wg, bg = rnd(1, 2 * heads, width, scale=0.5).to(dt), torch.cat([rnd(2, heads) - 1, rnd(3, heads) + 2])
    nw = rnd(4, inner, scale=0.1) + 1
    h = {s: rnd(10 + s, n, width).to(dt) for s, n in LENGTHS.items()}
    proj = {s: rnd(20 + s, n, stride).to(dt) for s, n in LENGTHS.items()}
    state = {"S": torch.full((5, heads, dim, vdim), float("nan")).cuda(), "n": torch.full((5, heads, dim), float("nan")).cuda(),
             "m": torch.full((5, heads), float("nan")).cuda()}
    both = {s: torch.cat([proj[s], torch.nn.functional.pad(h[s], (0, 0))], 1) for s in LENGTHS}      # a step's rows: proj | h

    def step(plan, rows):
        pr, hh = rows[:, :stride].contiguous(), rows[:, stride:].contiguous()
        gates = ops.mlstm_gates(hh, wg.cuda(), bg.cuda(), heads, cap)
        o = ops.mlstm_scan(pr, 0, qk, 2 * qk, gates, state, plan, heads, dim, vdim, 1e-6)
        return ops.gated_group_norm(o, pr, 2 * qk + inner, nw.cuda(), heads, eps, dt, gate_first=False, gate="sigmoid")

    got = feed(step, both, dt, stride + width)
    for s, n in LENGTHS.items():
        x, g = f64(proj[s]), f64(h[s]) @ f64(wg).T + f64(bg)
        log_i, log_f = P.soft_cap(g[:, :heads], cap), P.log_sigmoid(P.soft_cap(g[:, heads:], cap))
        q = x[:, :qk].reshape(n, heads, dim) * dim ** -0.5
        k, v = x[:, qk:2 * qk].reshape(n, heads, dim), x[:, 2 * qk:2 * qk + inner].reshape(n, heads, vdim)
        o = np.stack([P.rms_unit(P.mlstm_recurrence(q[:, a], k[:, a], v[:, a], log_i[:, a], log_f[:, a]), eps)
                      for a in range(heads)], 1).reshape(n, inner)
        close(got[s], o * f64(nw) * P.sigmoid(x[:, 2 * qk + inner:2 * qk + 2 * inner]), OP_TOL[dtype])


def test_the_matrix_memory_keeps_a_token_from_far_back(ops):
    """Forget gates near one, one early token written with a large input gate and read 600 tokens later with its own key."""
    T, dim, vdim = 640, 16, 8
    proj = torch.zeros(T, 2 * dim + 2 * vdim)
    proj[:, :dim] = rnd(1, T, dim, scale=0.05)
    proj[:, dim:2 * dim] = rnd(2, T, dim, scale=0.05)
    proj[:, 2 * dim:2 * dim + vdim] = rnd(3, T, vdim)
    proj[20, dim:2 * dim] = 3.0
    proj[20, 2 * dim:2 * dim + vdim] = 50.0
    proj[620, :dim] = 3.0
    # (a log forget gate that is a power of two: the running maximum then falls by exact steps in float32, where a value
    # like 1e-4 would be rounded the same way 600 times over and the maximum would drift by 6e-5)
    gates = torch.stack([torch.full((T,), -6.0), torch.full((T,), -2.0 ** -13)], 1)
    gates[20, 0] = 4.0
    state = {"S": torch.zeros(1, 1, dim, vdim).cuda(), "n": torch.zeros(1, 1, dim).cuda(), "m": torch.zeros(1, 1).cuda()}
    got = ops.mlstm_scan(proj.cuda(), 0, dim, 2 * dim, gates.cuda(), state, plan_of([(0, 0, T)]), 1, dim, vdim, 1e-6)
    x = f64(proj)
    want = P.mlstm_recurrence(x[:, :dim] * dim ** -0.5, x[:, dim:2 * dim], x[:, 2 * dim:2 * dim + vdim], f64(gates[:, 0]), f64(gates[:, 1]))
    assert want[620].min() > 40.0
    close(got, want, 3e-5)


@pytest.mark.parametrize("pieces", [1, 2, 5, None])
@pytest.mark.parametrize("heads, dim, vdim", [(2, 16, 24), (1, 40, 136), (1, 160, 72)])
def test_mlstm_in_pieces_side_by_side_equals_one_walk(ops, pieces, heads, dim, vdim):
    """Two sequences of unequal length, one of them on top of a carried state (its running maximum not zero); the shorter
    one ends before the last pieces begin.  Key sizes of every register layout, a last tile of a few value columns, and
    the count of pieces that the library picks itself (None)."""
    lengths = (300, 70)
    qk, inner = heads * dim, heads * vdim
    rows = rnd(1, sum(lengths), 2 * qk + inner, scale=0.7)
    gates = torch.cat([rnd(2, sum(lengths), heads, scale=2.0) - 1.0, -torch.nn.functional.softplus(rnd(3, sum(lengths), heads) - 2.0)], 1)
    first = {"S": rnd(4, 2, heads, dim, vdim), "n": rnd(5, 2, heads, dim), "m": rnd(6, 2, heads).abs() + 0.5}
    state = {k: v.clone().cuda() for k, v in first.items()}
    plan = plan_of([(0, 0, lengths[0]), (1, 9, lengths[1])])
    got = f64(ops.mlstm_scan(rows.cuda(), 0, qk, 2 * qk, gates.cuda(), state, plan, heads, dim, vdim, 1e-6, pieces=pieces))
    x, g, at = f64(rows), f64(gates), 0
    for i, n in enumerate(lengths):
        for a in range(heads):
            S = np.zeros((dim, vdim)) if i == 0 else f64(first["S"][1, a])
            nn = np.zeros(dim) if i == 0 else f64(first["n"][1, a])
            m = 0.0 if i == 0 else float(first["m"][1, a])
            for t in range(at, at + n):
                q, k = x[t, a * dim:(a + 1) * dim] * dim ** -0.5, x[t, qk + a * dim:qk + (a + 1) * dim]
                v = x[t, 2 * qk + a * vdim:2 * qk + (a + 1) * vdim]
                m_new = max(g[t, heads + a] + m, g[t, a])
                keep, take = math.exp(g[t, heads + a] + m - m_new), math.exp(g[t, a] - m_new)
                S, nn, m = keep * S + take * np.outer(k, v), keep * nn + take * k, m_new
                want = (S.T @ q) / (max(abs(nn @ q), math.exp(-m)) + 1e-6)
                assert np.abs(got[t, a * vdim:(a + 1) * vdim] - want).max() < 3e-5 * max(1.0, np.abs(want).max()), (i, a, t)
            assert np.abs(f64(state["S"][i, a]) - S).max() < 3e-5 * max(1.0, np.abs(S).max())
            assert np.abs(f64(state["n"][i, a]) - nn).max() < 3e-5 * max(1.0, np.abs(nn).max()) and abs(float(state["m"][i, a]) - m) < 1e-5
        at += n


# ------------------------------------------------------------------------------ minGRU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 50, 320])
def test_mingru_over_steps(ops, dtype, width):
    part = -(-width // 8) * 8
    bz, bx = rnd(1, width), rnd(2, width, scale=0.5)
    data = {s: rnd(10 + s, n, 3 * part, scale=2.0) for s, n in LENGTHS.items()}
    state = torch.full((5, width), float("nan")).cuda()
    got = feed(lambda plan, rows: ops.mingru(rows, 0, part, 2 * part, bz.cuda(), bx.cuda(), state, plan, width, DT[dtype]),
               data, torch.float32, 3 * part)
    for s, n in LENGTHS.items():
        x = f64(data[s])
        z, c = P.sigmoid(x[:, :width] + f64(bz)), P.mingru_candidate(x[:, part:part + width] + f64(bx))
        S, want = np.zeros(width), np.zeros((n, width))
        for t in range(n):
            S = (1 - z[t]) * S + z[t] * c[t]
            want[t] = S * P.silu(x[t, 2 * part:2 * part + width])
        close(got[s], want, OP_TOL[dtype])


@pytest.mark.parametrize("pieces", [1, 2, 7])
def test_mingru_in_pieces_side_by_side_equals_one_walk(ops, pieces):
    """Two sequences of unequal length, one of them on top of carried state; the candidate's two branches both taken."""
    width, lengths = 72, (700, 130)
    bz, bx = rnd(1, width), rnd(2, width, scale=0.5)
    rows = rnd(3, sum(lengths), 3 * width, scale=2.0).cuda()
    first = rnd(4, 2, width).cuda()
    state = first.clone()
    plan = plan_of([(0, 0, lengths[0]), (1, 5, lengths[1])])
    got = ops.mingru(rows, 0, width, 2 * width, bz.cuda(), bx.cuda(), state, plan, width, torch.float32, pieces=pieces)
    x, at = f64(rows), 0
    for i, n in enumerate(lengths):
        S = np.zeros(width) if i == 0 else f64(first[1])
        z, c = P.sigmoid(x[at:at + n, :width] + f64(bz)), P.mingru_candidate(x[at:at + n, width:2 * width] + f64(bx))
        assert (x[at:at + n, width:2 * width] + f64(bx) < 0).any() and (x[at:at + n, width:2 * width] + f64(bx) >= 0).any()
        for t in range(n):
            S = (1 - z[t]) * S + z[t] * c[t]
            assert np.abs(f64(got[at + t]) - S * P.silu(x[at + t, 2 * width:])).max() < 2e-5
        assert np.abs(f64(state[i]) - S).max() < 2e-5
        at += n


@pytest.mark.parametrize("pieces", [1, None])
def test_mingru_keeps_a_token_from_far_back(ops, pieces):
    """Gates shut but for one early token: every later state is that token's candidate, 600 tokens on and through the
    pieces of a long step; a second sequence opens its gate late and forgets what it held."""
    width, n = 40, 640
    rows = torch.zeros(2 * n, 3 * width)
    rows[:, :width] = -18.0                                    # gates shut: z = 1.5e-8
    rows[:, width:2 * width] = rnd(1, 2 * n, width)            # candidates that are never taken
    rows[:, 2 * width:] = 1.0
    rows[5, :width], rows[5, width:2 * width] = 18.0, torch.linspace(-3, 3, width)
    rows[n + 600, :width], rows[n + 600, width:2 * width] = 18.0, 2.0
    zeros = torch.zeros(width).cuda()
    state = torch.full((2, width), float("nan")).cuda()
    got = f64(ops.mingru(rows.cuda(), 0, width, 2 * width, zeros, zeros, state, plan_of([(0, 0, n), (1, 0, n)]), width,
                         torch.float32, pieces=pieces))
    held = P.mingru_candidate(np.linspace(-3, 3, width)) * float(P.silu(np.array(1.0)))
    assert np.abs(got[5:n] - held).max() < 1e-4 and np.abs(got[:5]).max() < 1e-6
    assert np.abs(got[n + 600:] - 2.5 * float(P.silu(np.array(1.0)))).max() < 1e-4 and np.abs(got[n:n + 600]).max() < 1e-4


# ------------------------------------------------------------------------------ attention with a distance penalty and a sink
def attention_steps(ops, dtype, heads, kv, hd, vd, window, steps, qkv_of, scale, slopes, sinks):
    """Feeds sequences step by step through the paged cache (pages taken in a scrambled order, NaN in every page
    before) and returns the outputs per sequence."""
    need = CacheNeed("window", kv, hd, window, 0, 0 if vd == hd else vd)
    cache = SequenceCache([(need, None)], [None], 4096, None, DT[dtype], "cuda")
    cache.groups[0].pages._free = np.random.default_rng(0).permutation(cache.n_pages).tolist()
    view = cache.views[0]
    view.k.fill_(float("nan"))
    view.v.fill_(float("nan"))
    n_seq = len(steps[0])
    slots = [cache.open() for _ in range(n_seq)]
    outs = [[] for _ in range(n_seq)]
    at = [0] * n_seq
    for news in steps:
        live = [(i, n) for i, n in enumerate(news) if n > 0]
        entries = [(slots[i], n) for i, n in live]
        tails = cache.reserve(entries)
        host = build_step([(s, [0] * n, []) for s, n in entries], cache.lengths, [cache.groups[0].table], cache.max_blocks, tails=tails)
        plan = StepPlan(host, torch.from_numpy(host.packed).cuda())
        if plan.has_tails:
            ops.clear_tails(cache.groups[0], plan.tails[0])
        qkv = torch.cat([qkv_of(i)[at[i]:at[i] + n] for i, n in live]).to(DT[dtype]).cuda().contiguous()
        out = ops.attention(qkv, view, plan, heads, kv, hd, scale, window, DT[dtype], store=True, keep_first=0, value_dim=vd,
                            slopes=slopes, sinks=sinks)
        cache.commit(entries)
        row = 0
        for i, n in live:
            outs[i].append(out[row:row + n])
            at[i] += n
            row += n
    cache.check()
    return [torch.cat(o) for o in outs]


def plain_attention_rows(qkv, heads, kv, hd, vd, window, scale, slopes, sinks):
    qkv = f64(qkv)
    T, per = qkv.shape[0], heads // kv
    q = qkv[:, :heads * hd].reshape(T, heads, hd)
    k = qkv[:, heads * hd:(heads + kv) * hd].reshape(T, kv, hd)
    v = qkv[:, (heads + kv) * hd:].reshape(T, kv, vd)
    out = np.zeros((T, heads, vd))
    for i in range(T):
        lo = max(0, i - window + 1)
        for a in range(heads):
            s = (k[lo:i + 1, a // per] @ q[i, a]) * scale
            if slopes is not None:
                s = s - slopes[a] * (i - np.arange(lo, i + 1))
            top = s.max() if sinks is None else max(s.max(), sinks[a])
            e = np.exp(s - top)
            out[i, a] = (e @ v[lo:i + 1, a // per]) / (e.sum() + (0.0 if sinks is None else math.exp(sinks[a] - top)))
    return out.reshape(T, heads * vd)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv, hd, vd, window", [(8, 2, 64, 64, 44), (6, 3, 24, 40, 33), (2, 1, 64, 64, 130), (4, 4, 32, 32, 64),
                                                      (2, 2, 16, 16, 1), (3, 1, 12, 10, 9), (10, 2, 16, 16, 100), (1, 1, 128, 128, 70)])
@pytest.mark.parametrize("bias", ["both", "slopes", "sinks"])
def test_attention_with_a_distance_penalty_and_a_sink(ops, dtype, heads, kv, hd, vd, window, bias):
    """Prompts of unequal length, portions on top of a cache, one token each; windows shorter and longer than a
    page; head sizes with and without a tensor-core kernel; the slopes of the design, sinks of both signs."""
    lengths = (290, 7, 140)
    width = (heads + kv) * hd + kv * vd
    data = [rnd(20 + i, n, width).to(DT[dtype]) for i, n in enumerate(lengths)]
    steps = [[200, 3, 70], [1, 1, 1], [1, 1, 1], [80, 2, 60], [1, 0, 1], [7, 0, 7]]
    scale = 0.9 / math.sqrt(hd)
    slopes = torch.tensor([P.slope(a, heads) for a in range(heads)]) if bias != "sinks" else None
    sinks = rnd(9, heads, scale=2.0) if bias != "slopes" else None
    got = attention_steps(ops, dtype, heads, kv, hd, vd, window, steps, lambda i: data[i], scale,
                          None if slopes is None else slopes.float().cuda(), None if sinks is None else sinks.cuda())
    for g, d in zip(got, data):
        want = plain_attention_rows(d, heads, kv, hd, vd, window, scale, None if slopes is None else f64(slopes),
                                    None if sinks is None else f64(sinks))
        close(g, want, OP_TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("prompt", [True, False])
def test_one_marked_key_is_seen_exactly_inside_the_window_and_pays_for_its_distance(ops, dtype, prompt):
    """One key matches the queries and carries a value of 100, every other value is 0, every other score about 0.  A query
    that sees the marked key from distance r reads 100 e^(a - slope r) / (e^(a - slope r) + the others + the sink), and
    exactly 0 where the window has passed the key.  Head 0 pays 0.05 a position and has a sink of weight one; head 1 pays
    nothing and its sink is negligible.  The marked key is placed at the first position, at a page's edge, and far back;
    in a prompt's rows and in rows decoded one by one."""
    heads, kv, hd, window = 2, 1, 32, 90
    T = 330
    slopes = torch.tensor([0.05, 0.0])
    sinks = torch.tensor([0.0, -30.0])
    for marked in (0, 63, 64, 191):       # (63 | 64: a page's last and first row)
        def qkv_of(_):
            qkv = rnd(marked, T, (heads + 2 * kv) * hd, scale=0.1)
            qkv[:, :heads * hd] += 6.0 * torch.ones(hd).repeat(heads)               # every query points along ones
            qkv[marked, heads * hd:(heads + kv) * hd] = 6.0                         # the marked key too
            qkv[:, (heads + kv) * hd:] = 0.0
            qkv[marked, (heads + kv) * hd:] = 100.0
            return qkv
        steps = [[T]] if prompt else [[marked + 2]] + [[1]] * (T - marked - 2)
        scale = 7.0 / (36.0 * hd)                                                   # the marked key's score is about 7
        got = f64(attention_steps(ops, dtype, heads, kv, hd, hd, window, steps, qkv_of, scale, slopes.cuda(), sinks.cuda())[0])
        for i in (marked, marked + 1, marked + window - 1, marked + window, marked + window + 1, T - 1):
            if i < T:
                seen = 0 <= i - marked < window
                for a in range(heads):
                    value = got[i, a * hd]
                    assert (value > 5.0) if seen else (abs(value) < 1e-2), (marked, i, a, seen, value)
        near, far = marked + 1, marked + window - 1
        if far < T:
            assert got[near, 0] > 90.0 and got[far, 0] < 50.0          # e^(7 - 0.05 * 89) against up to 90 others and the sink
            assert got[near, hd] > 90.0 and got[far, hd] > 80.0        # e^7 against up to 90 others


def test_a_sink_alone_in_the_denominator_halves_a_lone_keys_weight(ops):
    """The first token of a sequence sees one key: without a sink it reads that value whole, with a sink equal to its score half."""
    hd = 16
    qkv = torch.zeros(1, 3 * hd)
    qkv[0, 2 * hd:] = 8.0
    for sink, want in ((None, 8.0), (0.0, 4.0), (math.log(3.0), 2.0)):
        sinks = None if sink is None else torch.tensor([sink]).cuda()
        got = attention_steps(ops, "float32", 1, 1, hd, hd, 5, [[1]], lambda i: qkv, 1.0, torch.tensor([0.3]).cuda(), sinks)[0]
        assert abs(float(got[0, 0]) - want) < 1e-5


# ------------------------------------------------------------------------------ whole models through the engine
@pytest.fixture(scope="module")
def engines(folders):
    return {(name, dtype): E.Engine.from_folder(folders[name], dtype=dtype, max_tokens=2048)
            for name in folders for dtype in ("float32", "bfloat16")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["sos_a", "sos_b", "sos_c"])
def test_prompts_decoding_portions_and_batches_equal_the_plain_model(engines, plains, name, dtype):
    eng, m = engines[(name, dtype)], plains[name]
    vocab = m.cfg["vocab"]
    seqs = U.sequences(m, 10, (200, 1, 40, 97, 2))
    refs = [P.forward(m, s) for s in seqs]
    for prompts in ([len(s) for s in seqs], [150, 1, 1, 30, 1]):
        got, _ = run_batch(eng, seqs, prompts)
        assert max(U.row_error(g, r) for g, r in zip(got, refs)) < U.TOL[dtype]
    each_alone = [run_batch(eng, [s], [min(len(s), 33)])[0][0] for s in seqs]          # alone: no neighbour changes a row
    assert max(U.row_error(g, r) for g, r in zip(each_alone, refs)) < U.TOL[dtype]
    from_the_first = run_batch(eng, [seqs[2]], [1])[0][0]                              # one token at a time from the first
    assert U.row_error(from_the_first, refs[2]) < U.TOL[dtype]
    slot, at, rows = eng.open(), 0, []
    for n in (2, 5, 64, 3, 2, 30, 94):                                                 # portions of one sequence
        rows.append(eng.step([(slot, seqs[0][at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    eng.close(slot)
    assert U.row_error(np.concatenate(rows), refs[0]) < U.TOL[dtype]
    eng.ops.check()
    eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


def test_in_32_bit_a_row_does_not_depend_on_the_batch_or_the_cut(engines):
    eng = engines[("sos_a", "float32")]
    seqs = [U.ids(70 + i, 300, n) for i, n in enumerate((90, 31, 64))]
    together, _ = run_batch(eng, seqs, [60, 31, 1])
    for i, s in enumerate(seqs):
        alone, _ = run_batch(eng, [s], [len(s)])
        assert np.abs(alone[0] - together[i]).max() < 2e-5 * np.abs(alone[0]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_window_with_slots_used_again(folders, plains, dtype):
    """A small cache: sequences decoded far past the window hold few pages, and the next batch gets the
    slots, state rows and pages that the batch before it left (filled with NaN in between)."""
    eng, m = E.Engine.from_folder(folders["sos_a"], dtype=dtype, max_tokens=384), plains["sos_a"]
    for round_ in range(2):
        seqs = U.sequences(m, 200 * round_, (330, 90))
        got, slots = run_batch(eng, seqs, [3, 70])
        assert sorted(slots) == [0, 1]
        assert max(U.row_error(g, P.forward(m, s)) for g, s in zip(got, seqs)) < U.TOL[dtype]
        for g in eng.cache.groups:
            for t in g.k + g.v:
                t.fill_(float("nan"))
        for state in eng.cache.states:
            for t in state.values():
                t.fill_(float("nan"))
    assert max(g.pages.size for g in eng.cache.groups) == 6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_takes_the_recurrences_in_pieces(folders, plains, dtype):
    eng, m = E.Engine.from_folder(folders["sos_b"], dtype=dtype, max_tokens=1024), plains["sos_b"]
    seq = U.sequences(m, 77, (512,))[0]
    got, _ = run_batch(eng, [seq], [511])
    assert U.row_error(got[0], P.forward(m, seq)) < U.TOL[dtype]


def test_graph_replay_equals_launch_by_launch(folders):
    seqs = [U.ids(300 + i, 300, n) for i, n in enumerate((40, 75, 9))]
    outs = []
    for graphs in (True, False):
        eng = E.Engine.from_folder(folders["sos_a"], dtype="float32", max_tokens=1024, cuda_graphs=graphs)
        assert eng.cuda_graphs == graphs
        outs.append(run_batch(eng, seqs, [20, 60, 1])[0])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_session(folders, plains, dtype):
    for name in ("sos_a", "sos_b"):
        m = plains[name]
        session = E.Session(folders[name], None, max_batch_size=3, dtype=dtype, max_tokens=2048)
        prompts = U.sequences(m, 50, (5, 23, 1, 9))
        got = session.generate_batch(prompts, steps=8, temperature=0.0)
        want = [P.generate(m, p, 8) for p in prompts]
        if dtype == "float32":
            assert got == want
        else:       # a near tie may fall the other way in bfloat16: the first tokens agree, and most of the rest
            assert [g[0] for g in got] == [w[0] for w in want]
            assert sum(a == b for g, w in zip(got, want) for a, b in zip(g, w)) >= 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_model_folder(folders, plains, tmp_path, dtype):
    """bin/trace_run picks the model by config.json: each request whole, then unequal requests together and decoded
    together, their slots given back at their ends."""
    from test_replay_gpu import Replay
    m = plains["sos_b"]
    vocab = m.cfg["vocab"]
    seqs = {f"q{i}": s for i, s in enumerate(U.sequences(m, 400, (130, 1, 47)))}
    refs = {k: P.forward(m, s) for k, s in seqs.items()}
    rp = Replay(folders["sos_b"], dtype, tmp_path, sum(len(s) for s in seqs.values()))
    for k, s in seqs.items():
        got = rp.step([(k + "w", s, list(range(len(s))))], end=[k + "w"]).reshape(len(s), vocab)
        assert U.row_error(got, refs[k]) < U.TOL[dtype]
    fed = {k: max(1, len(s) - 20) for k, s in seqs.items()}
    rows = {k: [] for k in seqs}
    out = rp.step([(k, s[:fed[k]], list(range(fed[k]))) for k, s in seqs.items()], end=[k for k, s in seqs.items() if fed[k] == len(s)])
    at = 0
    for k in seqs:
        rows[k].append(out.reshape(-1, vocab)[at:at + fed[k]])
        at += fed[k]
    while any(fed[k] < len(s) for k, s in seqs.items()):
        live = [k for k, s in seqs.items() if fed[k] < len(s)]
        out = rp.step([(k, [seqs[k][fed[k]]], [0]) for k in live], end=[k for k in live if fed[k] + 1 == len(seqs[k])]).reshape(-1, vocab)
        for r, k in enumerate(live):
            rows[k].append(out[r:r + 1])
            fed[k] += 1
    rp.close()
    for k in seqs:
        assert U.row_error(np.concatenate(rows[k]), refs[k]) < U.TOL[dtype]


def test_the_command_line_generates_greedily(folders, plains):
    """bin/ember picks the model by config.json: a prompt's greedy tokens in 32-bit, and a batch of two prompts."""
    import os
    import subprocess
    import sys
    m = plains["sos_a"]
    prompt = U.sequences(m, 900, (7,))[0]
    cli = [sys.executable, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "ember")]
    r = subprocess.run(cli + [folders["sos_a"], "-", "1", "prompt", " ".join(map(str, prompt)), "-mt", "5", "-t", "0", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == P.generate(m, prompt, 5)
    other = U.sequences(m, 901, (3,))[0]
    r = subprocess.run(cli + [folders["sos_a"], "-", "1", "batch", "--batch-prompts", " ".join(map(str, prompt)), " ".join(map(str, other)),
                              "-mt", "3", "--temperature", "0", "--dtype", "float32", "-mbs", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "Output: " + " ".join(map(str, P.generate(m, other, 3))) in r.stdout
