"""Nimelorn on the device against the plain float64 implementation (plain_nimelorn.py): each mechanism alone, the replay
schedules (whole; the last tokens one by one; unequal batches one after another, so that slots and pages are used again;
prompts in pieces down to two tokens beside single tokens), long decoding past block edges and page borders, first tokens,
planted keys at the attention kernels under a block mask, the recurrence kernel alone, greedy generation through the engine."""
import numpy as np
import pytest
import torch

import plain_nimelorn as plain
import tiny_nimelorn as tiny
import trace_util as tu
from plain_lfm3 import load_folder

pytestmark = pytest.mark.gpu

COS = {"float32": 0.999999, "bfloat16": 0.95}       # (bfloat16: what a gap at the bound of tiny.upper_limit leaves)
LENGTHS = [1, 2, 7, 16, 23, 40, 70, 5, 13, 33, 64, 65, 131]


def requests_for(name, lengths=LENGTHS):
    return {f"r{i}": tiny.prompt(name, n, salt=i) for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("nimelorn_models")
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = tiny.make_folder(root, name, dtype)
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def replayers(folders):
    from xpu_serve_b200.engine.model import load_model
    from xpu_serve_b200.engine.replay import Replayer
    made = {}

    def get(name, dtype, max_tokens=1024):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Replayer(load_model(folders(name, dtype), dtype=dtype), max_tokens, None)
        return made[key]
    return get


_REFS = {}
CLOSE_CALL = {"float32": 1e-5, "bfloat16": 0.015}
NOISE = {"float32": 1e-7, "bfloat16": 2.0 ** -9}


def reference(folder, requests, dtype="float32", factors=None):
    """{(request, position): float64 logits}, memoised per folder and request. A token whose choice of experts is a
    close call at this precision may choose otherwise on the device, and every later position of its sequence may see
    that (through the recurrence and the keys): those are left out. The position vector's angle is the float32 product
    of position and frequency in the design, so the oracle forms it so too (everything else is float64).

    `factors` takes, per place, how much more than the typical place the oracle's own logits there move under a
    relative perturbation of every weight of the size of the precision under test (NOISE; at least 1). With random weights the recurrence's output is now and
    then a small difference of large terms (a query nearly orthogonal to the few keys that carry the state's weight),
    which the norm over the head then scales up; rounding moves such a place by that much more too."""
    cfg, W = load_folder(folder)
    out = {}
    for rid, toks in requests.items():
        key = (folder, tuple(toks))
        if key not in _REFS:
            logits = plain.forward(cfg, W, toks, angle_bits=32)
            moved = np.zeros(len(toks))
            for draw in (1, 2, 3):           # (three draws: one alone may leave a touchy place unmoved by chance)
                rng = np.random.default_rng(draw)
                W2 = {k: np.asarray(v, dtype=np.float64) * (1.0 + NOISE[dtype] * rng.standard_normal(np.asarray(v).shape)) for k, v in W.items()}
                moved = np.maximum(moved, np.abs(plain.forward(cfg, W2, toks, angle_bits=32) - logits).max(-1))
            _REFS[key] = (logits, plain.router_margins(cfg, W, toks), np.maximum(moved / max(np.median(moved), 1e-300), 1.0))
        logits, margins, factor = _REFS[key]
        close = np.nonzero(margins < CLOSE_CALL[dtype])[0]
        for p in range(len(toks) if close.size == 0 else int(close[0])):
            out[(rid, p)] = logits[p]
            if factors is not None:
                factors[(rid, p)] = float(factor[p])
    return out


def weighted_gap(got, ref, factors):
    """tu.worst_gap with every place's gap divided by its factor: (largest, its place, lowest cosine, places whose
    factor is above 4, all gaps in descending order)."""
    scale = max(np.abs(v).max() for v in ref.values())
    worst, where, cos = 0.0, None, 1.0
    gaps = []
    assert set(got) == set(ref), f"places differ: {sorted(set(ref) ^ set(got))[:5]}"
    for key in sorted(ref):
        a, b = got[key].astype(np.float64), ref[key]
        assert np.isfinite(a).all(), f"non-finite logits at {key}"
        gap = np.abs(a - b).max() / scale / factors[key]
        gaps.append(gap)
        if gap > worst:
            worst, where = gap, key
        if factors[key] <= 4.0:
            cos = min(cos, float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300)))
    return worst, where, cos, sum(1 for k in ref if factors[k] > 4.0), sorted(gaps, reverse=True)


def check(name, dtype, steps, requests, replayers, folders, max_tokens=1024, replayer=None):
    rp = replayer or replayers(name, dtype, max_tokens)
    got = tu.collect(steps, tu.run_in_process(rp, steps), tiny.CONFIGS[name]["vocab"])
    factors = {}
    ref = reference(folders(name, dtype), requests, dtype, factors)
    ref = {k: v for k, v in ref.items() if k in got}
    assert len(ref) >= min(len(got), 8), "the test's first tokens are close calls of a router; pick other prompts"
    gap, where, cos, touchy, gaps = weighted_gap({k: v for k, v in got.items() if k in ref}, ref, factors)
    assert touchy <= len(ref) // 5, f"{touchy} of {len(ref)} places are badly conditioned; pick other weights"
    tol = tiny.upper_limit(name, dtype)
    print(f"GAP nimelorn {name} {dtype} steps={len(steps)} gap={gap:.3e} at {where} (factor {factors[where]:.1f}) cos={cos:.7f} "
          f"tol={tol:.1e} touchy={touchy}")
    if dtype == "float32":
        assert gap <= tol, f"{name} {dtype}: gap {gap:.3e} at {where}"
    else:
        # At 8 significant bits a place where the recurrence's output nearly cancels moves by more than three perturbed runs
        # of the oracle foretell: one place in fifty (at least one) may pass the bound, none four times the bound. A fault
        # in a mechanism moves most places (test_a_lost_part_is_caught).
        allowed = max(1, len(gaps) // 50)
        assert gap <= 4.0 * tol, f"{name} {dtype}: gap {gap:.3e} at {where}"
        assert len(gaps) <= allowed or gaps[allowed] <= tol, f"{name} {dtype}: {sum(g > tol for g in gaps)} places over {tol:.2e}"
    if dtype == "float32" or gaps[0] <= tol:          # (a place that was let pass the bound above has its own cosine)
        assert cos >= COS[dtype], f"{name} {dtype}: cosine {cos}"
    rp.cache.check()
    assert rp.cache.slots.held_count == 0 and rp.cache.tokens_held() == 0
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["blocked", "borrowed", "odd", "recurrent", "dense", "routed"])
def test_one_mechanism_alone(name, dtype, replayers, folders):
    """Single-mechanism models (the mixers without any feed-forward): a whole prompt, then the same with its tail token
    by token, then unequal requests together."""
    reqs = requests_for(name, [1, 2, 11, 37, 90])
    check(name, dtype, tu.whole_trace(reqs), reqs, replayers, folders)
    check(name, dtype, tu.tail_trace(reqs, tail=20), reqs, replayers, folders)
    check(name, dtype, tu.batch_trace(reqs, 3), reqs, replayers, folders)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole(name, dtype, replayers, folders):
    reqs = requests_for(name)
    check(name, dtype, tu.whole_trace(reqs), reqs, replayers, folders)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prefill_then_token_by_token(name, dtype, replayers, folders):
    reqs = requests_for(name)
    check(name, dtype, tu.tail_trace(reqs, tail=32), reqs, replayers, folders)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [3, 5, 13])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(name, batch, dtype, replayers, folders):
    """Batches of unequal requests against each alone; a later batch takes the slots and pages that the one before gave
    back (with the last tokens and recurrent states they held), in a cache that holds little more than one batch."""
    reqs = requests_for(name)
    check(name, dtype, tu.batch_trace(reqs, batch), reqs, replayers, folders, max_tokens=1280)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pieces", [(2, 3, 64, 5), (7, 64, 65, 129, 3, 16, 40), (130, 2)])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompts_in_pieces(name, pieces, dtype, replayers, folders):
    """Pieces of several sizes, down to two tokens, at page borders and across block edges, in steps that mix a later
    piece of one request with single tokens of others: a piece's first token finds its predecessor in the slot."""
    reqs = requests_for(name, [131, 2, 70, 23, 140, 64, 9])
    check(name, dtype, tu.pieces_trace(reqs, 4, pieces=pieces), reqs, replayers, folders)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("C", "bfloat16")])
def test_long_decoding(name, dtype, replayers, folders):
    """A short prompt and 200 tokens one by one: over every block edge and three page borders, with the recurrent state
    and the last token carried through every step; beside it a second request that ends early. (In bfloat16 only the
    configuration without experts: among 200 tokens a router's close call comes early, and everything behind it is left out.)"""
    reqs = {"long": tiny.prompt(name, 204, salt=3), "short": tiny.prompt(name, 30, salt=4)}
    check(name, dtype, tu.batch_trace(reqs, 2, prompt_frac=0.02), reqs, replayers, folders)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts(dtype, replayers, folders):
    """Prompts of 300 and 520 tokens beside one of 46 in one step, then single tokens: the recurrent layers cut the long
    ones into chunks that run side by side (the last ones partly filled), each sequence's state
    carried from chunk to chunk and on into the single tokens that follow."""
    from xpu_serve_b200.ops import lib as ops
    reqs = {"a": tiny.prompt("C", 306, salt=5), "b": tiny.prompt("C", 526, salt=6), "c": tiny.prompt("C", 46, salt=7)}
    seen = []
    real = ops.mlstm_scan
    ops.mlstm_scan = lambda *a, **k: (seen.append(a[-1] if len(a) == 18 else k.get("chunks")), real(*a, **k))[1]
    try:
        check("C", dtype, tu.batch_trace(reqs, 3, prompt_frac=0.985), reqs, replayers, folders, max_tokens=1280)
    finally:
        ops.mlstm_scan = real
    # (chunks of 64 tokens here: five, nine and one)
    assert any(c is not None and c[0].shape[0] == 5 + 9 + 1 for c in seen), "the long prompts did not take the chunked scan"


def test_every_product_on_the_tcgen05_kernel(folders, monkeypatch):
    """With the tcgen05 product forced for every number of rows, the squared ReLU runs in the up product's epilogue (C has
    widths in blocks of 8); whole prompts and single tokens against the oracle."""
    from xpu_serve_b200.engine.model import load_model
    from xpu_serve_b200.engine.replay import Replayer
    from xpu_serve_b200.ops import lib as ops
    monkeypatch.setenv("XS_MANY_ROWS_GEMM", "tcgen05")
    rp = Replayer(load_model(folders("C", "bfloat16"), dtype="bfloat16"), 1024, None)
    assert rp.model.rt.many_rows == "tcgen05"
    seen = []
    real = ops.gemm_tc
    monkeypatch.setattr(ops, "gemm_tc", lambda *a, **k: (seen.append((a[0].shape[0], k.get("epilogue"))), real(*a, **k))[1])
    reqs = requests_for("C", [70, 131, 9])
    check("C", "bfloat16", tu.tail_trace(reqs, tail=6), reqs, None, folders, replayer=rp)
    # whole prompts' rows (single tokens take the weight-streaming product, which has the activation in its epilogue too)
    assert (64, ops.EPI_RELU_SQ) in seen and (125, ops.EPI_RELU_SQ) in seen


def test_the_program_replays_a_trace(folders, tmp_path):
    """bin/trace_run over its standard input, in float32, against the oracle."""
    reqs = requests_for("C", [5, 40, 70])
    steps = tu.tail_trace(reqs, tail=4)
    folder = folders("C", "float32")
    got = tu.collect(steps, tu.run_program(folder, "float32", steps, str(tmp_path / "out"), 512, tiny.CONFIGS["C"]["vocab"]),
                     tiny.CONFIGS["C"]["vocab"])
    factors = {}
    ref = reference(folder, reqs, factors=factors)
    gap, where, cos, _, _ = weighted_gap(got, {k: v for k, v in ref.items() if k in got}, factors)
    assert gap <= 1e-5 and cos >= COS["float32"], (gap, where, cos)


def test_a_lost_part_is_caught(replayers, folders, monkeypatch):
    """The bounds see a block mask that is one position off, a predecessor that is forgotten between steps, a state that
    is not zeroed, and a shared unit that is left out."""
    from xpu_serve_b200.engine.model import load_model
    from xpu_serve_b200.engine.replay import Replayer
    from xpu_serve_b200.ops import lib as ops
    reqs = requests_for("C", [40, 70])
    steps = tu.tail_trace(reqs, tail=10)
    real_generic = ops.attention_generic

    def fresh(name, dtype):            # kernel by kernel, so that every launch goes through the functions patched below
        rp = Replayer(load_model(folders(name, dtype), dtype=dtype), 1024, None)
        rp.model.use_graphs = rp.model.use_prompt_graphs = False
        return rp

    def shifted(fn, at):
        def run(*a, **k):
            a = list(a)
            a[at] = a[at] - 1 if a[at] < 0 else a[at]      # a block of one position more
            return fn(*a, **k)
        return run

    rp32 = fresh("C", "float32")
    check("C", "float32", steps, reqs, replayers, folders, replayer=rp32)          # (sound before the fault is planted)
    monkeypatch.setattr(ops, "attention_generic", shifted(real_generic, 10))
    with pytest.raises(AssertionError):
        check("C", "float32", steps, reqs, replayers, folders, replayer=rp32)
    monkeypatch.undo()
    # the last token kept in the slot is what a later step's first token is paired with
    real_embed = ops.embed_pair

    def forgetful(table, pair, ids, positions, seq_of, cu, slots, last, *rest):
        last.zero_()
        return real_embed(table, pair, ids, positions, seq_of, cu, slots, last, *rest)

    rp16 = fresh("C", "bfloat16")
    monkeypatch.setattr(ops, "embed_pair", forgetful)
    with pytest.raises(AssertionError):
        check("C", "bfloat16", steps, reqs, replayers, folders, replayer=rp16)
    monkeypatch.undo()
    real_combine = ops.moe_combine
    monkeypatch.setattr(ops, "moe_combine", lambda rows, place, wts, y, top, shared=None, gate=None: real_combine(rows, place, wts, y, top))
    r1 = requests_for("routed", [40, 70])
    with pytest.raises(AssertionError):
        check("routed", "bfloat16", tu.whole_trace(r1), r1, replayers, folders, replayer=fresh("routed", "bfloat16"))
    monkeypatch.undo()
    rp = rp16
    for g in rp.cache.groups:
        if not hasattr(g, "pages"):                 # the groups of fixed-size state: opening a slot no longer zeroes it
            monkeypatch.setattr(g, "zero", lambda slots: None)
    tu.run_in_process(rp, steps)                                        # leaves states behind in the slots
    with pytest.raises(AssertionError):
        check("C", "bfloat16", steps, reqs, replayers, folders, replayer=rp)      # ... which the same slots now start from


# ------------------------------------------------------------------------- the attention kernels with planted keys
def plain_block_attention(q, keys, values, pos, scale, chunk, gate):
    """Float64 attention of one token's heads [H, D] at position `pos` over keys [n, G, D] and values [n, G, Dv]."""
    H, G = q.shape[0], keys.shape[1]
    lo = pos - pos % chunk
    out = np.zeros((H, values.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = scale * (keys[lo:pos + 1, g] @ q[h])
        e = np.exp(s - s.max())
        out[h] = (e / e.sum()) @ values[lo:pos + 1, g]
        if gate is not None:
            out[h] *= 1.0 / (1.0 + np.exp(-gate[h]))
    return out


@pytest.mark.parametrize("kernel,dtype", [("generic", torch.float32), ("generic", torch.bfloat16), ("mma", torch.bfloat16),
                                          ("mma split", torch.bfloat16), ("decode", torch.bfloat16), ("decode split", torch.bfloat16),
                                          ("tcgen05", torch.bfloat16)])
@pytest.mark.parametrize("chunk", [37, 64, 100, 1])
def test_attention_kernels_under_a_block_mask(kernel, dtype, chunk):
    """Queries of several sequences in one launch, pages in a shuffled order. For two queries, the first key of their own
    block, the last key of the block before, a key at a page's last place and one far back are made to dominate (the key
    is the query's direction, scaled), so leaving one out or letting one in changes the result by far more than the bound."""
    from xpu_serve_b200.ops import lib as ops
    torch.manual_seed(7)
    H, G, D, page = 4, 2, 64, 64
    lens = [300, 129, 64, 1]
    decode = kernel.startswith("decode")
    q_lens = [1, 1, 1, 1] if decode else [12, 1, 1, 1]
    if kernel == "tcgen05":
        if not ops.attention_tc_supports(D, page, H // G):
            pytest.skip("the tcgen05 kernel does not take this shape")
        q_lens = [140, 70, 9, 1]
    n_pages = sum(-(-n // page) for n in lens)
    order = torch.randperm(n_pages + 3)
    pool = torch.zeros(n_pages + 4, 2, G, page, D, dtype=dtype, device="cuda")
    table = torch.full((len(lens), 5), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(lens):
        for p in range(-(-n // page)):
            table[s, p] = int(order[at]); at += 1
    keys = [torch.randn(n, G, D) * 0.3 for n in lens]
    values = [torch.randn(n, G, D) for n in lens]
    T = sum(q_lens)
    q = torch.randn(T, H, D) * 0.3
    positions, seq_of = [], []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n)); seq_of += [s] * ql
    for s, t in ((0, q_lens[0] - 1), (1, q_lens[0] + q_lens[1] - 1)):
        pos = positions[t]
        lo = pos - pos % chunk
        for j in {3, 63, 64, lo, lo - 1, pos} - {-1}:
            if 0 <= j <= pos:
                direction = q[t, 1]
                keys[s][j, 0] = direction / direction.norm() * 6.0
    for s in range(len(lens)):
        k, v = keys[s].to(dtype), values[s].to(dtype)
        keys[s], values[s] = k.double().numpy(), v.double().numpy()
        for j in range(k.shape[0]):
            pool[int(table[s, j // page]), 0, :, j % page] = k[j].cuda()
            pool[int(table[s, j // page]), 1, :, j % page] = v[j].cuda()
    qd = q.to(dtype).cuda()
    gate = (torch.randn(T, H) * 2).to(dtype).cuda()
    out = torch.empty(T, H, D, dtype=dtype, device="cuda")
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    cu = dev([0] + list(np.cumsum(q_lens)))
    if kernel == "generic":
        ops.attention_generic(qd, pool, table.cuda(), dev(seq_of), dev(positions), gate, out, G, page, 0.9, -chunk)
    elif kernel == "tcgen05":
        ops.attention_tc(qd, pool, table.cuda(), cu, dev(lens), gate, out, len(lens), max(q_lens), G, page, 0.9, -chunk, max(lens))
    else:
        splits = 3 if "split" in kernel else 1
        scratch = torch.empty(ops.attention_mma_scratch_bytes(T * H, D, splits) + 16, dtype=torch.uint8, device="cuda") if splits > 1 else None
        ops.attention_mma(qd, pool, table.cuda(), cu, dev(lens), gate, out, scratch, len(lens), max(q_lens), G, page, 0.9,
                          -chunk, splits, bounded_waits=decode)
    torch.cuda.synchronize()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for t in range(T):
        ref = plain_block_attention(qd[t].double().cpu().numpy(), keys[seq_of[t]], values[seq_of[t]], positions[t], 0.9, chunk,
                                    gate[t].double().cpu().numpy())
        gap = np.abs(out[t].double().cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-3)
        assert gap < tol, (kernel, t, positions[t], gap)


# ------------------------------------------------------------------------------------------- the recurrence alone
def plain_mlstm(q, k, v, zi, zf, bi, bf, cap, S, n, m):
    """One head, float64, token by token from the state (S [D, Dv], n [D], m). Returns the outputs [T, Dv] and the state."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        i = cap * np.tanh((zi[t] + bi) / cap)
        z = cap * np.tanh((zf[t] + bf) / cap)
        f = -np.logaddexp(0.0, -z)
        m2 = max(f + m, i)
        a, b = np.exp(f + m - m2), np.exp(i - m2)
        S = a * S + b * np.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m2
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), np.exp(-m)) + 1e-6)
    return out, S, n, m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv", [(3, 10, 14), (2, 32, 32), (1, 64, 300), (2, 128, 40), (5, 1, 1), (1, 200, 40)])
def test_mlstm_kernel_alone(H, D, Dv, dtype):
    """Sequences of 1, 2, 9 and 70 tokens in one launch, in slots given in another order, from states that are not zero;
    then the same tokens one launch a token: outputs and states against the plain recurrence. Gates large enough that the
    running maximum moves and both branches of the denominator's maximum occur."""
    from xpu_serve_b200.ops import lib as ops
    rng = np.random.default_rng(H * 100 + D)
    q_lens, slots = [1, 2, 9, 70], [3, 0, 4, 1]
    T, Z, cap = sum(q_lens), ops.mlstm_copies(Dv), 6.0
    ld = 2 * H * D + H * Dv + 5
    proj = torch.from_numpy(rng.standard_normal((T, ld)) * 0.7).to(dtype)
    gates = torch.from_numpy(rng.standard_normal((T, 2 * H + 3)) * 5.0).float()
    bi, bf = torch.from_numpy(rng.uniform(-1, 1, H)).float(), torch.from_numpy(rng.uniform(0, 3, H)).float()
    S0 = torch.from_numpy(rng.standard_normal((6, H, D, Dv)) * 0.5).float()
    n0 = torch.from_numpy(rng.standard_normal((6, H, D)) * 0.5).float()
    m0 = torch.from_numpy(rng.uniform(-2, 4, (6, H))).float()
    nm0 = torch.cat([n0, m0[..., None]], -1)[:, :, None, :].repeat(1, 1, Z, 1).contiguous()
    cu = [0] + list(np.cumsum(q_lens))
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    scale = 0.37
    # whole pieces in one launch
    S, nm = S0.clone().cuda(), nm0.clone().cuda()
    y = torch.zeros(T, H * Dv, device="cuda")
    ops.mlstm_scan(proj.cuda(), 0, H * D, 2 * H * D, gates.cuda(), bi.cuda(), bf.cuda(), S, nm, dev(cu), dev(slots), y, H, D, Dv, cap, scale)
    # token by token
    S1, nm1 = S0.clone().cuda(), nm0.clone().cuda()
    y1 = torch.zeros(T, H * Dv, device="cuda")
    for s, (b, e) in enumerate(zip(cu[:-1], cu[1:])):
        for t in range(b, e):
            ops.mlstm_scan(proj[t:t + 1].cuda(), 0, H * D, 2 * H * D, gates[t:t + 1].cuda(), bi.cuda(), bf.cuda(), S1, nm1,
                           dev([0, 1]), dev([slots[s]]), y1[t:t + 1], H, D, Dv, cap, scale)
    torch.cuda.synchronize()
    P = proj.double().numpy()
    tol = 3e-5
    for s, (b, e) in enumerate(zip(cu[:-1], cu[1:])):
        for h in range(H):
            qh = P[b:e, h * D:(h + 1) * D] * scale
            kh = P[b:e, H * D + h * D:H * D + (h + 1) * D]
            vh = P[b:e, 2 * H * D + h * Dv:2 * H * D + (h + 1) * Dv]
            ref, Sr, nr, mr = plain_mlstm(qh, kh, vh, gates[b:e, h].double().numpy(), gates[b:e, H + h].double().numpy(),
                                          float(bi[h]), float(bf[h]), cap, S0[slots[s], h].double().numpy(),
                                          n0[slots[s], h].double().numpy(), float(m0[slots[s], h]))
            for got_y, got_S, got_nm in ((y, S, nm), (y1, S1, nm1)):
                g = got_y[b:e, h * Dv:(h + 1) * Dv].double().cpu().numpy()
                assert np.abs(g - ref).max() <= tol * max(np.abs(ref).max(), 1.0), (s, h)
                assert np.abs(got_S[slots[s], h].double().cpu().numpy() - Sr).max() <= tol * max(np.abs(Sr).max(), 1.0)
                for z in range(Z):
                    assert np.abs(got_nm[slots[s], h, z, :D].double().cpu().numpy() - nr).max() <= tol * max(np.abs(nr).max(), 1.0)
                    assert abs(float(got_nm[slots[s], h, z, D]) - mr) <= 1e-5 * max(abs(mr), 1.0)
    # slots that no sequence of the launch used are untouched
    for free in (2, 5):
        assert torch.equal(S[free].cpu(), S0[free]) and torch.equal(nm[free].cpu(), nm0[free])


@pytest.mark.parametrize("H,D,Dv,chunk", [(3, 10, 14, 7), (2, 64, 70, 128), (1, 128, 32, 50), (1, 130, 70, 64)])
def test_mlstm_kernel_in_chunks(H, D, Dv, chunk):
    """Sequences of 300, 46 and 520 tokens cut into chunks that run side by side (a pass from the empty state, the carry,
    a pass from each chunk's true state), from states that are not zero: outputs and end states against the plain
    recurrence run token by token. Forget gates near 0 and near 1 and input gates of both signs, so that the maximum is
    now carried from before the chunk, now set inside it."""
    from xpu_serve_b200.ops import lib as ops
    rng = np.random.default_rng(H + D + chunk)
    q_lens, slots = [300, 46, 520], [2, 0, 3]
    T, Z, cap, scale = sum(q_lens), ops.mlstm_copies(Dv), 6.0, 0.4
    ld = 2 * H * D + H * Dv
    proj = torch.from_numpy(rng.standard_normal((T, ld)) * 0.7).float()
    gates = torch.from_numpy(rng.standard_normal((T, 2 * H)) * 4.0).float()
    bi, bf = torch.from_numpy(rng.uniform(-1, 1, H)).float(), torch.from_numpy(rng.uniform(0, 3, H)).float()
    S0 = torch.from_numpy(rng.standard_normal((4, H, D, Dv)) * 0.5).float()
    n0 = torch.from_numpy(rng.standard_normal((4, H, D)) * 0.5).float()
    m0 = torch.from_numpy(rng.uniform(-2, 4, (4, H))).float()
    nm0 = torch.cat([n0, m0[..., None]], -1)[:, :, None, :].repeat(1, 1, Z, 1).contiguous()
    cu = [0] + list(np.cumsum(q_lens))
    rows, first = [], [0]
    for i, (b, e) in enumerate(zip(cu[:-1], cu[1:])):
        rows += [(i, t, min(chunk, e - t)) for t in range(b, e, chunk)]
        first.append(len(rows))
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    S, nm = S0.clone().cuda(), nm0.clone().cuda()
    y = torch.zeros(T, H * Dv, device="cuda")
    scratch = (dev(rows), dev(first), torch.empty(len(rows), H, D, Dv, device="cuda"), torch.empty(len(rows), H, Z, D + 2, device="cuda"))
    ops.mlstm_scan(proj.cuda(), 0, H * D, 2 * H * D, gates.cuda(), bi.cuda(), bf.cuda(), S, nm, dev(cu), dev(slots), y, H, D, Dv,
                   cap, scale, scratch)
    torch.cuda.synchronize()
    P = proj.double().numpy()
    tol = 1e-4
    for s, (b, e) in enumerate(zip(cu[:-1], cu[1:])):
        for h in range(H):
            ref, Sr, nr, mr = plain_mlstm(P[b:e, h * D:(h + 1) * D] * scale, P[b:e, H * D + h * D:H * D + (h + 1) * D],
                                          P[b:e, 2 * H * D + h * Dv:2 * H * D + (h + 1) * Dv], gates[b:e, h].double().numpy(),
                                          gates[b:e, H + h].double().numpy(), float(bi[h]), float(bf[h]), cap,
                                          S0[slots[s], h].double().numpy(), n0[slots[s], h].double().numpy(), float(m0[slots[s], h]))
            g = y[b:e, h * Dv:(h + 1) * Dv].double().cpu().numpy()
            assert np.abs(g - ref).max() <= tol * max(np.abs(ref).max(), 1.0), (s, h, np.abs(g - ref).max())
            assert np.abs(S[slots[s], h].double().cpu().numpy() - Sr).max() <= tol * max(np.abs(Sr).max(), 1.0)
            for z in range(Z):
                assert np.abs(nm[slots[s], h, z, :D].double().cpu().numpy() - nr).max() <= tol * max(np.abs(nr).max(), 1.0)
                assert abs(float(nm[slots[s], h, z, D]) - mr) <= 1e-4 * max(abs(mr), 1.0)
    assert torch.equal(S[1].cpu(), S0[1]) and torch.equal(nm[1].cpu(), nm0[1])       # a slot that no sequence used


def test_embedding_alone():
    """Two sequences in one launch, one from its first token and one going on behind a token kept in its slot: rows
    against the formula, and the slots' words afterwards."""
    from xpu_serve_b200.ops import lib as ops
    rng = np.random.default_rng(3)
    V, W, buckets, mp, mc, scale, eps = 50, 22, 13, 7, 5, 2.5, 1e-5
    table = torch.from_numpy(rng.standard_normal((V, W))).float()
    pair = torch.from_numpy(rng.standard_normal((buckets + 1, W))).float()
    w = torch.from_numpy(rng.uniform(0.5, 1.5, W)).float()
    f = 10000.0 ** (-2.0 * np.arange((W + 1) // 2) / W)
    toks = [[4, 9, 9, 30], [17, 2, 41]]
    starts, before = [0, 100], [0, 33]
    last = torch.zeros(6, 1, dtype=torch.int32)
    last[2, 0] = 33
    last[5, 0] = 11             # what an earlier user of this slot left: a first token must not read it
    slots = [5, 2]
    flat = [t for seq in toks for t in seq]
    pos = [starts[s] + i for s, seq in enumerate(toks) for i in range(len(seq))]
    seq_of = [s for s, seq in enumerate(toks) for _ in seq]
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    h = torch.zeros(len(flat), W, device="cuda")
    last_d = last.cuda()
    ops.embed_pair(table.cuda(), pair.cuda(), dev(flat), dev(pos), dev(seq_of), dev([0, 4, 7]), dev(slots), last_d,
                   torch.from_numpy(f).float().cuda(), w.cuda(), h, scale, buckets, mp, mc, eps)
    at = 0
    for s, seq in enumerate(toks):
        prev = before[s]
        for i, t in enumerate(seq):
            p = starts[s] + i
            row = buckets if p == 0 else (prev * mp + t * mc) % buckets
            x = table[t].double().numpy() * scale + pair[row].double().numpy()
            x[0::2] += np.sin(p * f)
            x[1::2] += np.cos(p * f)
            ref = plain.rms_norm(x, w.double().numpy(), eps)
            assert np.abs(h[at].double().cpu().numpy() - ref).max() < 2e-5, (s, i)
            prev = t
            at += 1
    assert int(last_d[5, 0]) == 30 and int(last_d[2, 0]) == 41 and int(last_d[0, 0]) == 0


# --------------------------------------------------------------------------------------------------------- generation
def plain_greedy(cfg, W, prompt, n):
    seq, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = plain.forward(cfg, W, seq, angle_bits=32)[-1]
        order = np.argsort(-logits)
        margins.append(float(logits[order[0]] - logits[order[1]]) / float(np.abs(logits).max()))
        out.append(int(order[0]))
        seq.append(out[-1])
    return out, margins


@pytest.mark.parametrize("precision,name", [("f32", "A"), ("bf16", "C")])
@pytest.mark.parametrize("chunk", [None, 16])
def test_greedy_generation_through_the_engine(folders, chunk, precision, name):
    """The framework's own entry point and scheduler: three unequal prompts as one batch (with `chunk`, prompts in
    pieces of 16 tokens), greedy, against the plain implementation run token by token. In float32 every token must be
    the oracle's; in bfloat16 a sequence is followed until the oracle's own choice is a near tie."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    dtype = {"f32": "float32", "bf16": "bfloat16"}[precision]
    folder = folders(name, dtype)
    cfg, W = load_folder(folder)
    kw = {} if chunk is None else {"prefill_chunk": chunk}
    engine = Engine(folder, precision=precision, ctx=256, max_batch=8, **kw)
    prompts = [tiny.prompt(name, n, salt=i) for i, n in enumerate((3, 41, 18))]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), 9, []) for p in prompts])
    followed = 0
    for p, r in zip(prompts, res):
        assert r.finish == "length" and len(r.tokens) == 9
        if precision == "f32":
            want, margins = plain_greedy(cfg, W, p, 9)
            if min(margins) > 1e-4:
                assert r.tokens == want
                followed += 9
            continue
        seq = list(p)
        for t in r.tokens:
            logits = plain.forward(cfg, W, seq, angle_bits=32)[-1]
            order = np.argsort(-logits)
            if (logits[order[0]] - logits[order[1]]) / np.abs(logits).max() < 0.03:
                break
            assert t == int(order[0]), (len(seq) - len(p), t, int(order[0]))
            followed += 1
            seq.append(t)
    assert followed >= 3, "near ties everywhere; pick other prompts"
    engine.stepper.cache.check()
    assert engine.stepper.cache.slots.held_count == 0


@pytest.mark.parametrize("chunk", [None, 16])
def test_generation_with_experts_in_bfloat16_follows_replay(folders, replayers, chunk):
    """With experts the oracle's choice of experts is a close call too often at 16 bits to follow it for long, so here
    the engine (prompts as captured graphs or in pieces of 16 tokens; decode graphs, one step ahead of the loop) is held
    against trace replay of the same tokens (plain launches): two paths through the same kernels. A token may differ only
    where replay's own two best logits are within a hundredth of the largest."""
    from xpu_serve_b200 import GenerateRequest, SamplingParams
    from xpu_serve_b200.engine.engine import Engine
    folder = folders("B", "bfloat16")
    kw = {} if chunk is None else {"prefill_chunk": chunk}
    engine = Engine(folder, precision="bf16", ctx=256, max_batch=8, **kw)
    prompts = [tiny.prompt("B", n, salt=i) for i, n in enumerate((3, 41, 18))]
    res = engine.generate([GenerateRequest(p, SamplingParams(temperature=0.0), 9, []) for p in prompts])
    rp = replayers("B", "bfloat16")
    same = 0
    for p, r in zip(prompts, res):
        assert r.finish == "length" and len(r.tokens) == 9
        logits = rp.run_step({"step": 0, "entries": [{"id": "g", "tokens": p, "want": [0, len(p) - 1]}], "end": []})[-1]
        for i, t in enumerate(r.tokens):
            order = np.argsort(-logits)
            if t != int(order[0]):
                assert (logits[order[0]] - logits[order[1]]) / np.abs(logits).max() < 1e-2, (i, t, int(order[0]))
                break
            same += 1
            logits = rp.run_step({"step": i + 1, "entries": [{"id": "g", "tokens": [t], "want": [0]}], "end": []})[0]
        rp.run_step({"step": 99, "entries": [], "end": ["g"]})
    assert same >= 20
    engine.stepper.cache.check()
    assert engine.stepper.cache.slots.held_count == 0 and rp.cache.slots.held_count == 0


def test_the_command_line_generates(folders):
    """`bin/xpu-serve run` on a Nimelorn folder in float32, greedy: the plain implementation's tokens."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders("C", "float32")
    cfg, W = load_folder(folder)
    prompt = tiny.prompt("C", 11, salt=91)
    want, margins = plain_greedy(cfg, W, prompt, 8)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "xpu-serve"), "run", folder, "--prompt", " ".join(map(str, prompt)),
                        "--max-tokens", "8", "--temperature", "0", "--precision", "f32", "--ctx", "128"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    res = json.loads(p.stdout.strip().splitlines()[-1])
    assert len(res["tokens"]) == 8
    if min(margins) > 1e-4:
        assert res["tokens"] == want
    else:                                   # up to the oracle's own first near tie
        k = next(i for i, m in enumerate(margins) if m <= 1e-4)
        assert res["tokens"][:k] == want[:k]
