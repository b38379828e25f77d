"""The Vizonex decoder on the GPU against the plain restatement: each mechanism's kernels alone, with
weights or inputs made so that a fault shows (a key just outside a chunk, a sink that outweighs the keys,
a state that has to survive hundreds of tokens, a kept input at a portion's start), then whole models (four
tiny configurations of unlike sizes) whole, token by token, in portions, in mixed batches on few pages and
slots, and through the generation entry point."""
import math

import numpy as np
import pytest
import torch

import plain_vizonex as plain
import replay_util as ru
from tiny import random_ids
from tiny_vizonex import SHARPEN, TINY, make_folder, reference_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from tokenizer_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, what="", tol=None):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    tol = tol if tol is not None else (2e-5 if dtype == torch.float32 else 2e-2)
    bound = tol * max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all() and err <= bound, f"{what}: max |diff| {err:.3e} > {bound:.3e}"


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def batch_of(counts):
    """Device metadata of a step whose request r brings counts[r] rows: (row_req, q_start)."""
    row_req = [r for r, n in enumerate(counts) for _ in range(n)]
    starts = [0]
    for n in counts:
        starts.append(starts[-1] + n)
    return ints(row_req), ints(starts)


# ---- the short convolution, its kept inputs across steps ------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps,residual,activation,bias", [
    (50, 4, True, None, False), (96, 1, True, None, False), (384, 3, False, "silu", True), (1030, 7, False, "silu", True),
    (64, 2, True, None, False)])
def test_short_convolution_over_portions_gives_what_the_whole_sequences_give(channels, taps, residual, activation, bias, dtype):
    """Three requests of unlike lengths on slots 3, 0 and 2 of four, fed in portions down to one row: the rows
    before a portion's start come from the slot, and rows before a sequence's start are zeros although the
    slots hold what an earlier request left."""
    o = ops()
    lengths, slots = [37, 5, 90], [3, 0, 2]
    extra = 8                                           # columns in front of the channels, as in a stacked product
    xs = [rnd(n, extra + channels, seed=10 + i, dtype=dtype) for i, n in enumerate(lengths)]
    w = rnd(channels, taps, seed=20, scale=0.6)
    b = rnd(channels, seed=21) if bias else None
    off = 12
    state = torch.full((4, off + (taps - 1) * channels + 4), 7.0, device=DEV)    # stale numbers everywhere
    for s in slots:
        state[s].zero_()                                # what opening a request does
    want = []
    for x in xs:
        y = plain.causal_convolution(x[:, extra:].double().cpu(), w.double().cpu(), b.double().cpu() if bias else None)
        y = plain.silu(y) if activation else y
        want.append(y + x[:, extra:].double().cpu() if residual else y)
    got = [torch.empty(n, channels, device=DEV) for n in lengths]
    done = [0, 0, 0]
    sizes = [1, 2, 9, 1, 1, 30, 3, 64]
    step = 0
    while any(d < n for d, n in zip(done, lengths)):
        take = [min(sizes[(step + r) % len(sizes)], n - d) for r, (d, n) in enumerate(zip(done, lengths))]
        if step % 3 == 0:
            take = [min(1, t) for t in take]              # a step of single tokens: the kept inputs move in the same launch
        live = [r for r in range(3) if take[r] and (step + r) % 4 != 3]      # a request sits out now and then
        if not live:
            step += 1
            continue
        single = all(take[r] == 1 for r in live)
        rows = torch.cat([xs[r][done[r]:done[r] + take[r]] for r in live])
        rows = torch.cat([rows, torch.full((2, rows.shape[1]), float("nan"), dtype=dtype, device=DEV)])   # padding rows
        row_req, q_start = batch_of([take[r] for r in live])
        row_req = torch.cat([row_req, ints([-1, -1])])
        out = torch.full((rows.shape[0], channels), float("nan"), device=DEV)
        slot_of = ints([slots[r] for r in live])
        o.short_conv(rows, extra, channels, w, b, state, off, row_req, q_start, slot_of, out, activation=activation,
                     residual=residual, shift=single)
        if not single:
            o.short_conv_state(rows, extra, channels, taps, state, off, q_start, slot_of)
        at = 0
        for r in live:
            got[r][done[r]:done[r] + take[r]] = out[at:at + take[r]]
            at += take[r]
            done[r] += take[r]
        step += 1
    for r in range(3):
        close(got[r], want[r], torch.float32, f"request {r}", tol=2e-5 if dtype == torch.float32 else 1e-5)
    assert float(state[1].min()) == 7.0                  # a slot of no request is left alone
    if taps > 1:                                         # what is kept: the last taps - 1 inputs, oldest first
        kept = state[slots[2], off:off + (taps - 1) * channels].view(taps - 1, channels)
        close(kept, xs[2][-(taps - 1):, extra:], torch.float32, "kept inputs", tol=0.0 if dtype == torch.float32 else 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels,taps", [(320, 4), (72, 2), (128, 3), (50, 3)])
def test_short_convolution_in_steps_of_thousands_of_rows(channels, taps, dtype):
    """Steps of 2,437 and of 360 rows (the kernel's runs of rows begin inside requests and straddle their borders),
    then one of single tokens."""
    o = ops()
    lengths, slots = [1100 + 120 + 1, 37 + 120 + 1, 1300 + 120 + 1], [1, 2, 0]
    xs = [rnd(n, channels, seed=25 + i, dtype=dtype) for i, n in enumerate(lengths)]
    w, b = rnd(channels, taps, seed=28, scale=0.6), rnd(channels, seed=29)
    state = torch.zeros(3, (taps - 1) * channels, device=DEV)
    want = [plain.silu(plain.causal_convolution(x.double().cpu(), w.double().cpu(), b.double().cpu())) for x in xs]
    done = [0, 0, 0]
    for take in ([1100, 37, 1300], [120, 120, 120], [1, 1, 1]):
        rows = torch.cat([xs[r][done[r]:done[r] + take[r]] for r in range(3)])
        row_req, q_start = batch_of(take)
        out = torch.full((rows.shape[0], channels), float("nan"), dtype=dtype, device=DEV)
        single = take == [1, 1, 1]
        o.short_conv(rows, 0, channels, w, b, state, 0, row_req, q_start, ints(slots), out, activation="silu", shift=single)
        if not single:
            o.short_conv_state(rows, 0, channels, taps, state, 0, q_start, ints(slots))
        at = 0
        for r in range(3):
            close(out[at:at + take[r]], want[r][done[r]:done[r] + take[r]], dtype, f"request {r}")
            at += take[r]
            done[r] += take[r]
    kept = state[slots[1]].view(taps - 1, channels)
    close(kept, xs[1][-(taps - 1):], torch.float32, "kept inputs", tol=0.0 if dtype == torch.float32 else 1e-6)


# ---- both sublayers' outputs, each scaled by its vector, added; the norm behind -------------------------
@pytest.mark.parametrize("width", [50, 320, 2048, 8192, 9001])
@pytest.mark.parametrize("form", ["one bf16", "two bf16", "f32 and partials"])
def test_scaled_outputs_are_added_and_the_sum_is_normed(width, form):
    o = ops()
    n = 9
    x = rnd(n, width, seed=30, scale=2.0)
    v1, v2 = rnd(width, seed=31), rnd(width, seed=32)
    if form == "f32 and partials":
        a, b = rnd(n, width, seed=33), rnd(3, n, width, seed=34)
        b_sum = b.double().sum(dim=0)
    else:
        a, b = rnd(n, width, seed=33, dtype=torch.bfloat16), rnd(n, width, seed=34, dtype=torch.bfloat16)
        b_sum = b.double()
    terms = [(a, v1)] if form == "one bf16" else [(a, v1), (b, v2)]
    want_x = x.double() + a.double() * v1.double() + (0 if form == "one bf16" else b_sum * v2.double())
    gain = rnd(width, seed=35) + 1.0
    for normed in (False, True):
        x_run = x.clone()
        if normed:
            out = torch.full((n, width), float("nan"), device=DEV)
            o.scaled_add_norm(x_run, terms, gain, 1e-5, out)
            close(out, plain.rms(want_x, 1e-5) * gain.double(), torch.float32, "the norm of the sum")
        else:
            o.scaled_add_norm(x_run, terms)
        close(x_run, want_x, torch.float32, "the sum")


# ---- learned positions ----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [50, 320])
def test_embedding_adds_the_rows_of_a_position_table(width, dtype):
    o = ops()
    table, positions = rnd(77, width, seed=40, dtype=dtype), rnd(300, width, seed=41, dtype=dtype)
    ids, pos, req = [5, 76, 0, 9, 9, 3], [0, 299, 17, 1, 2, 0], [0, 0, 1, 2, 2, -1]
    out = torch.full((6, width), float("nan"), device=DEV)
    o.embed_positions(ints(ids), ints(pos), ints(req), table, positions, out)
    want = table.double()[ids[:5]] + positions.double()[pos[:5]]
    close(out[:5], want, torch.float32, "embedding + position", tol=1e-6)


# ---- queries and keys normed over the whole projection, a temperature a head ----------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim", [(6, 2, 64, 128), (3, 3, 10, 20), (4, 1, 32, 16), (1, 1, 24, 24)])
def test_whole_projection_norms_and_head_temperatures_in_the_cache_write(heads, kv, dim, vdim, dtype):
    """One root mean square over ALL of a token's query lanes (not one a head), one over all key lanes; heads of
    unlike sizes in the input make a norm taken head by head differ by far more than the tolerance."""
    o = ops()
    n, extra, row = 7, 4, -(-max(dim, vdim) // 16) * 16
    width = heads * dim + kv * (dim + vdim)
    proj = rnd(n, extra + width + 1, seed=50)
    lanes = torch.arange(heads * dim, device=DEV) // dim
    proj[:, extra:extra + heads * dim] *= (1.0 + 3.0 * lanes)              # head h is 1 + 3 h times larger
    proj[:, extra + heads * dim:extra + (heads + kv) * dim] *= 0.01        # eps matters for the keys
    q_gain, k_gain, temp = rnd(heads * dim, seed=51) + 1.0, rnd(kv * dim, seed=52) + 1.0, rnd(heads, seed=53) + 1.5
    eps = 1e-4
    pos, slots, req = [0, 1, 2, 0, 9, 3, 4], [4, 9, 2, 7, 0, 5, 3], [0, 0, 0, 1, 2, -1, 3]
    q = torch.full((n, heads * row), float("nan"), dtype=dtype, device=DEV)
    k_pool = torch.full((10, kv, row), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((10, kv, row), float("nan"), dtype=dtype, device=DEV)
    o.qkv_rotate_store(proj, extra, None, None, 0, ints(pos), ints(slots), ints(req), q, k_pool, v_pool, heads, kv, dim,
                       vdim, row, q_gain=q_gain, k_gain=k_gain, eps=eps, temp=temp)
    p = proj.double().cpu()[:, extra:extra + width]
    want_q = (plain.rms(p[:, :heads * dim], eps) * q_gain.double().cpu()).view(n, heads, dim) * temp.double().cpu()[None, :, None]
    want_k = (plain.rms(p[:, heads * dim:(heads + kv) * dim], eps) * k_gain.double().cpu()).view(n, kv, dim)
    want_v = p[:, (heads + kv) * dim:].view(n, kv, vdim)
    got_q = q.view(n, heads, row).float().cpu()
    for t in [t for t in range(n) if req[t] >= 0]:
        close(got_q[t, :, :dim], want_q[t], dtype, "queries")
        close(k_pool[slots[t]][:, :dim], want_k[t], dtype, "keys")
        close(v_pool[slots[t]][:, :vdim], want_v[t], dtype, "values")
        assert float(got_q[t, :, dim:].abs().max() if row > dim else 0) == 0
    assert torch.isnan(k_pool[slots[5]].float()).all()
    if heads > 1:                                       # a norm a head would give every head the same size
        per_head = plain.rms(p[:, :heads * dim].view(n, heads, dim), eps)
        assert float((per_head[0] * q_gain.double().cpu().view(heads, dim) * temp.double().cpu()[:, None] - want_q[0]).abs().max()) > 0.5


# ---- chunks and the sink in every attention kernel ------------------------------------------------------
def paged(lengths, kv, row, page, dtype, seed):
    """Keys and values of requests of these lengths, dense, and pools and tables to scatter them into (pages in a
    shuffled order, two spare)."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    pools = [torch.full((n_pages * page, kv, row), float("nan"), dtype=dtype) for _ in range(2)]
    tables = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    dense = [[torch.randn(n, kv, row, generator=g).to(dtype), torch.randn(n, kv, row, generator=g).to(dtype)] for n in lengths]
    return pools, tables, dense, order


def scatter(pools, tables, dense, order, page):
    for r, (k, v) in enumerate(dense):
        for b in range(-(-k.shape[0] // page)):
            pg = order.pop()
            tables[r, b] = pg
            rows = slice(b * page, min(k.shape[0], (b + 1) * page))
            pools[0][pg * page:pg * page + rows.stop - rows.start] = k[rows]
            pools[1][pg * page:pg * page + rows.stop - rows.start] = v[rows]


def run_attention(kernel, q, pools, tables, row_req, pos, spans, heads, kv, row, page, scale, sink, chunk):
    from tokenizer_b200.parts.attention import RowTiles
    o = ops()
    out = torch.full((len(pos), heads * row), float("nan"), dtype=q.dtype, device=DEV)
    args = (q.to(DEV).view(len(pos), -1), pools[0].to(DEV), pools[1].to(DEV), out, tables.to(DEV), ints(row_req), ints(pos))
    if kernel == "generic":
        o.paged_attention_generic(*args, heads, kv, row, page, None, scale, sink=sink, chunk=chunk)
    elif kernel == "decode":
        o.decode_attention(*args, heads, kv, row, page, None, scale, sink=sink, chunk=chunk)
    else:
        note = RowTiles(o.WIDE_TILE_ROWS if kernel == "wide" else o.PREFILL_TILE_ROWS)
        words = np.zeros(note.capacity(len(pos), len(spans)), dtype=np.int32)
        counts = np.array([m for _, _, m in spans], dtype=np.int32)
        firsts = np.concatenate(([0], np.cumsum(counts)[:-1])).astype(np.int32)
        n_tiles = note.fill(words, firsts, counts, np.array([f for _, f, _ in spans], dtype=np.int32), False)
        tiles = torch.tensor(words, device=DEV).view(-1, 2)
        run = o.attention_tcgen05 if kernel == "wide" else o.prefill_attention
        run(*args, tiles, n_tiles, heads, kv, row, page, None, scale, sink=sink, chunk=chunk)
    return out.view(len(pos), heads, row).float().cpu()


def plain_rows(q, dense, row_req, pos, heads, kv, scale, sink, chunk):
    """Every row's output from `plain.sink_chunk_attention`, one call a request over its whole length (rows that
    are not in the step ask with zeros and are dropped)."""
    out = torch.zeros(q.shape, dtype=torch.float64)
    ones = torch.ones(heads, dtype=torch.float64)
    for r, (k, v) in enumerate(dense):
        mine = [t for t in range(q.shape[0]) if row_req[t] == r]
        if not mine:
            continue
        queries = torch.zeros(k.shape[0], heads, q.shape[2], dtype=torch.float64)
        queries[[pos[t] for t in mine]] = q[mine].double()
        full = plain.sink_chunk_attention(queries, k.double(), v.double(), scale, ones, sink.double().cpu(), chunk)
        out[mine] = full[[pos[t] for t in mine]]
    return out


ATTENTION_CASES = [
    ("generic", torch.float32, 3, 3, 48, 160), ("generic", torch.bfloat16, 4, 2, 144, 37), ("generic", torch.float32, 2, 1, 32, 1),
    ("generic", torch.float32, 2, 1, 16, None),
    ("decode", torch.bfloat16, 4, 2, 32, 160), ("decode", torch.bfloat16, 16, 1, 64, 37), ("decode", torch.bfloat16, 2, 2, 128, 256),
    ("decode", torch.bfloat16, 2, 2, 48, None),
    ("tiles", torch.bfloat16, 3, 3, 48, 37), ("tiles", torch.bfloat16, 4, 2, 80, 160), ("tiles", torch.bfloat16, 2, 2, 16, 1),
    ("wide", torch.bfloat16, 4, 2, 128, 160), ("wide", torch.bfloat16, 6, 3, 128, 37), ("wide", torch.bfloat16, 2, 1, 64, 128),
    ("wide", torch.bfloat16, 2, 1, 64, None)]


@pytest.mark.parametrize("kernel,dtype,heads,kv,row,chunk", ATTENTION_CASES)
def test_chunk_edges_and_the_sink_in_every_attention_kernel(kernel, dtype, heads, kv, row, chunk):
    """For every request's last row, the key just before its chunk and the first key inside get scores that stand
    out and values of their own: the one must be missing from the output, the other must dominate it.  Each head
    has a sink of its own size; head 0's outweighs a hundred ordinary keys.  Requests end right behind, on and before a chunk's edge, and one of them is a single token (the
    first token of a sequence sees itself and the sink)."""
    page, size = 16, chunk or 100
    lengths = [3 * size + 2, 2 * size + 1, 1, 4 * size] if size > 1 else [70, 33, 1, 16]
    pools, tables, dense, order = paged(lengths, kv, row, page, dtype, seed=60)
    scale = 1.0 / math.sqrt(row)
    if kernel == "decode":
        row_req, pos, spans = [0, 1, 2, 3], [n - 1 for n in lengths], None
    else:
        take = [min(n, 130) for n in lengths]
        spans = [(r, n - m, m) for r, (n, m) in enumerate(zip(lengths, take))]
        row_req = [r for r, _, m in spans for _ in range(m)]
        pos = [first + i for _, first, m in spans for i in range(m)]
    q = rnd(len(pos), heads, row, seed=61, dtype=dtype).cpu()
    last = [t for t in range(len(pos)) if t + 1 == len(pos) or row_req[t + 1] != row_req[t]]
    for t in last:
        start = pos[t] - pos[t] % size if chunk else 0
        k, v = dense[row_req[t]]
        direction = q[t, 0].float() / q[t, 0].float().norm()
        if start > 0:
            k[start - 1, 0] = (direction * 40.0).to(dtype)
            v[start - 1, 0] = 50.0
        if start < pos[t]:
            k[start, 0] = (direction * 20.0).to(dtype)
            v[start, 0] = -9.0
    scatter(pools, tables, dense, order, page)
    sink = torch.linspace(-1.0, 2.0, heads)
    sink[0] = 6.0
    got = run_attention(kernel, q, pools, tables, row_req, pos, spans, heads, kv, row, page, scale, sink.to(DEV), chunk)
    want = plain_rows(q, dense, row_req, pos, heads, kv, scale, sink, chunk)
    assert torch.isfinite(got).all()
    bound = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((got - want).abs().max()) <= bound * max(1.0, float(want.abs().max()))
    # the sink matters: without it the outputs are others (a first token alone would return its own value whole)
    none = plain_rows(q, dense, row_req, pos, heads, kv, scale, torch.full((heads,), -1e30), chunk)
    assert float((none - want).abs().max()) > 0.5
    # the edge matters: seeing the key just outside would pull head 0 of the planted rows to its value
    if chunk and chunk > 1:
        open_ = plain_rows(q, dense, row_req, pos, heads, kv, scale, sink, None)
        assert float((open_ - want).abs().max()) > 5.0


@pytest.mark.parametrize("kernel,dtype,row", [("generic", torch.float32, 48), ("decode", torch.bfloat16, 64),
                                              ("tiles", torch.bfloat16, 48), ("wide", torch.bfloat16, 128)])
def test_a_far_key_among_hundreds_is_found(kernel, dtype, row):
    """Without chunks, key 3 of 1,500 carries the last query's own direction: its value must come back whole, from
    whichever page it lies on."""
    heads, kv, page, n = 2, 1, 16, 1500
    pools, tables, dense, order = paged([n], kv, row, page, dtype, seed=70)
    take = 1 if kernel == "decode" else 200
    spans = [(0, n - take, take)]
    row_req, pos = [0] * take, list(range(n - take, n))
    q = rnd(take, heads, row, seed=71, dtype=dtype).cpu()
    direction = q[-1, 1].float() / q[-1, 1].float().norm()
    dense[0][0][3, 0] = (direction * 60.0).to(dtype)
    dense[0][1][3, 0] = 25.0
    scatter(pools, tables, dense, order, page)
    sink = torch.zeros(heads)
    got = run_attention(kernel, q, pools, tables, row_req, pos, spans, heads, kv, row, page, 1.0 / math.sqrt(row),
                        sink.to(DEV), None)
    assert float((got[-1, 1] - 25.0).abs().max()) < 0.3


# ---- the selective state-space recurrence ---------------------------------------------------------------
def scan_in_steps(o, xbc, proj, dt_at, dt_bias, a_log, skip, heads, groups, vdim, n_state, lengths, slots, sizes, n_slots=4,
                  state=None, segments=None):
    """`mamba2_scan` over requests laid end to end in `xbc` / `proj`, fed in portions of `sizes` in turn; every
    request's matrices live in its slot.  `segments`: into how many segments that run side by side a request's
    rows of a step are cut (None: the kernel's own choice).  Returns y laid out like xbc, and the state arena."""
    firsts = [sum(lengths[:r]) for r in range(len(lengths))]
    if state is None:
        state = torch.full((n_slots, heads * vdim * n_state + 5), 3.0, device=DEV)      # stale numbers
        for s in slots:
            state[s].zero_()
    y = torch.full((xbc.shape[0], heads * vdim), float("nan"), device=DEV)
    done, step = [0] * len(lengths), 0
    while any(d < n for d, n in zip(done, lengths)):
        take = [min(sizes[(step + r) % len(sizes)], n - d) for r, (d, n) in enumerate(zip(done, lengths))]
        live = [r for r in range(len(lengths)) if take[r]]
        rows = torch.cat([torch.arange(firsts[r] + done[r], firsts[r] + done[r] + take[r]) for r in live]).to(DEV)
        _, q_start = batch_of([take[r] for r in live])
        out = torch.full((rows.shape[0], heads * vdim), float("nan"), device=DEV)
        o.mamba2_scan(xbc[rows].contiguous(), proj[rows].contiguous(), dt_at, dt_bias, a_log, skip, heads, groups, vdim,
                      n_state, state, q_start, ints([slots[r] for r in live]), out, segments=segments)
        y[rows] = out
        for r in live:
            done[r] += take[r]
        step += 1
    return y, state


@pytest.mark.parametrize("segments", [None, 1, 3, 16])
@pytest.mark.parametrize("proj_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,vdim,n_state", [(8, 2, 32, 32), (3, 3, 10, 6), (2, 1, 5, 40), (2, 2, 40, 256),
                                                       (4, 1, 64, 128), (1, 1, 1, 1)])
def test_state_space_recurrence_in_portions_and_batches_against_the_plain_one(heads, groups, vdim, n_state, proj_dtype,
                                                                              segments):
    """Three requests of unlike lengths, whole in one step and then in portions down to one token on other slots:
    both must give what the plain recurrence gives from a zero state, also where a request's rows of a step run
    as segments side by side (segments of 16 and 48 rows, requests with fewer segments than asked for, portions
    that continue from matrices that are not zero)."""
    o = ops()
    lengths = [45, 3, 130]
    total, inner = sum(lengths), heads * vdim
    xbc = rnd(total, inner + 2 * groups * n_state, seed=80, scale=0.7)
    dt_at = 3
    proj = rnd(total, dt_at + heads + 2, seed=81, dtype=proj_dtype)
    dt_bias, a_log, skip = rnd(heads, seed=82, scale=0.5), rnd(heads, seed=83, scale=0.5) - 1.0, rnd(heads, seed=84) + 1.0
    want = torch.zeros(total, inner, dtype=torch.float64)
    x64, p64 = xbc.double().cpu(), proj.double().cpu()
    at = 0
    for n in lengths:
        rows = slice(at, at + n)
        dt = plain.softplus(p64[rows, dt_at:dt_at + heads] + dt_bias.double().cpu())
        for h in range(heads):
            g = h // (heads // groups)
            B = x64[rows, inner + g * n_state:inner + (g + 1) * n_state]
            C = x64[rows, inner + (groups + g) * n_state:inner + (groups + g + 1) * n_state]
            want[rows, h * vdim:(h + 1) * vdim] = plain.selective_state_space(
                x64[rows, h * vdim:(h + 1) * vdim], B, C, dt[:, h], torch.exp(a_log.double().cpu()[h]), skip.double().cpu()[h])
        at += n
    args = (o, xbc, proj, dt_at, dt_bias, a_log, skip, heads, groups, vdim, n_state, lengths)
    whole, state_a = scan_in_steps(*args, [2, 0, 3], [1000], segments=segments)
    close(whole, want, torch.float32, "whole", tol=5e-5)
    pieces, state_b = scan_in_steps(*args, [1, 3, 0], [1, 2, 17, 1, 1, 40, 5], segments=segments)
    close(pieces, want, torch.float32, "in portions", tol=5e-5)
    size = heads * vdim * n_state
    close(state_b[1, :size], state_a[2, :size], torch.float32, "the matrices after the last token", tol=5e-5)
    assert float(state_a[1].min()) == 3.0 and float(state_a[2, size:].abs().max()) == 0.0      # nothing else is touched


@pytest.mark.parametrize("segments", [1, 4, 7])
def test_what_a_token_wrote_far_back_is_still_in_the_state(segments):
    """Almost no decay and B, C at right angles from token to token: what token 2 wrote along its own direction
    comes back when token 700 asks along it, across steps of 1, 2, 300 and more tokens and across the segments
    of a step; a state lost at a step's or a segment's edge gives zeros, and a slot used again starts from zero."""
    o = ops()
    heads, groups, vdim, n_state, total = 2, 1, 8, 16, 701
    inner = heads * vdim
    xbc = torch.zeros(total, inner + 2 * n_state, device=DEV)
    for t in range(total):
        xbc[t, inner + 1 + t % (n_state - 1)] = 1.0                  # B: e1 .. e15 in turn
        xbc[t, inner + n_state + 1 + (t + 5) % (n_state - 1)] = 1.0  # C likewise
        xbc[t, :inner] = 0.01
    marker = torch.arange(1, inner + 1, device=DEV).float()
    xbc[2, inner:] = 0.0
    xbc[2, inner] = 1.0                                              # token 2 alone writes along e0
    xbc[2, :inner] = marker
    xbc[700, inner + n_state:] = 0.0
    xbc[700, inner + n_state] = 1.0                                  # token 700 reads along e0
    xbc[700, :inner] = 0.0
    proj = torch.full((total, heads), 0.5413, device=DEV)           # softplus -> dt = 1
    zeros = torch.zeros(heads, device=DEV)
    a_log = torch.full((heads,), -30.0, device=DEV)                  # decay exp(-1e-13 dt) = 1
    y, state = scan_in_steps(o, xbc, proj, 0, zeros, a_log, zeros, heads, groups, vdim, n_state, [total], [1],
                             [1, 2, 300, 1, 397], segments=segments)
    dt = math.log1p(math.exp(0.5413))
    assert torch.allclose(y[700], marker * dt, rtol=1e-5)
    # the same slot for a new request: opened (zeroed), it knows nothing of the marker
    state[1].zero_()
    y2, _ = scan_in_steps(o, xbc[3:], proj[3:], 0, zeros, a_log, zeros, heads, groups, vdim, n_state, [total - 3], [1], [1000],
                          state=state, segments=segments)
    assert float(y2[700 - 3].abs().max()) == 0.0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,parts", [(256, 2), (30, 3), (10, 1), (2560, 4), (64, 64), (4100, 1)])
def test_gate_then_norm_in_equal_parts_of_the_row(inner, parts, out_dtype):
    o = ops()
    n = 6
    y, gain = rnd(n, inner, seed=90, scale=2.0), rnd(inner, seed=91) + 1.0
    proj = rnd(n, 5 + inner, seed=92)
    out = torch.full((n, inner), float("nan"), dtype=out_dtype, device=DEV)
    req = ints([0, 0, 1, -1, 2, 2])
    o.mamba2_out_norm(y, proj, 5, gain, 1e-3, parts, req, out)
    gated = y.double().cpu() * plain.silu(proj.double().cpu()[:, 5:])
    want = plain.rms(gated.view(n, parts, inner // parts), 1e-3).reshape(n, inner) * gain.double().cpu()
    live = [0, 1, 2, 4, 5]
    close(out[live], want[live], out_dtype, "gate, norm in parts")
    if parts > 1:                                       # the norm of the whole row is something else
        assert float((plain.rms(gated, 1e-3) * gain.double().cpu() - want).abs().max()) > 1e-2


# ---- the router and the experts' activation -------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,count,keep", [(8, 3, 2, 1), (8, 3, 4, 2), (6, 2, 3, 2), (3, 3, 1, 1), (4, 1, 4, 1),
                                                    (64, 6, 8, 3), (5, 2, 1, 1), (6, 2, 6, 3)])
def test_choice_on_corrected_scores_inside_the_best_groups_and_weights_without_the_correction(experts, top, count, keep, dtype):
    """Corrections as large as the scores themselves, some of them negative enough that every choice score of a
    group is below zero (a masked expert that counted as 0 would then win): the chosen experts are the plain
    router's, their shares the plain scores times the constant, every other share zero."""
    o = ops()
    n, hidden = 61, 50
    h = rnd(n, hidden, seed=100, dtype=dtype)
    w = rnd(experts, hidden, seed=101, scale=0.4)
    correction = rnd(experts, seed=102, scale=0.6) - 0.8
    share = torch.full((n, experts + 1), float("nan"), device=DEV)
    o.moe_route(h, w, experts, top, "one", share, score="sigmoid", correction=correction, groups=count, keep=keep, scale=2.5)
    weights = {"router": w.double().cpu(), "correction": correction.double().cpu()}
    r = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": count, "keep": keep}}
    chosen, shares = plain.route(h.double().cpu(), weights, "", r)
    want = torch.zeros(n, experts, dtype=torch.float64).scatter(1, chosen, shares)
    close(share[:, :experts], want, torch.float32, "shares")
    assert int((share[:, :experts] != 0).sum()) == n * top and float((share[:, experts] - 1.0).abs().max()) == 0.0


def test_experts_outside_the_kept_groups_are_out_even_when_every_choice_score_is_negative():
    """Corrections below -1 make every choice score negative; the best group is the one that is least so, and its
    experts are chosen although an expert counted as 0 would rank above them."""
    o = ops()
    n, hidden, experts = 17, 24, 6
    h, w = rnd(n, hidden, seed=103), rnd(experts, hidden, seed=104, scale=0.3)
    correction = torch.tensor([-5.0, -5.2, -2.0, -2.1, -3.0, -9.0], device=DEV)
    share = torch.full((n, experts), float("nan"), device=DEV)
    o.moe_route(h, w, experts, 2, None, share, score="sigmoid", correction=correction, groups=3, keep=1, scale=1.0)
    s = plain.sigmoid(h.double().cpu() @ w.double().cpu().t())
    want = torch.zeros(n, experts, dtype=torch.float64)
    want[:, 2:4] = s[:, 2:4]
    close(share, want, torch.float32, "shares of the second group's experts")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_activation_of_the_experts_lanes(dtype):
    """Gates and ups far beyond the limits on both sides; the shared expert's lanes have a limit of their own."""
    o = ops()
    n, experts, ff, sff, limit, shared_limit = 23, 5, 6, 10, 1.5, 0.75
    inner = experts * ff + sff
    gu = rnd(n, 2 * inner, seed=110, dtype=dtype, scale=2.0)
    share = rnd(n, experts + 1, seed=111).abs()
    share[:, experts] = 1.0
    act = torch.empty(n, inner, dtype=dtype, device=DEV)
    o.moe_gate(gu, share, act, experts, ff, True, activation="clamped_swish", limit=limit, shared_limit=shared_limit, alpha=1.702)
    g64 = gu.double().cpu()
    lane_expert = torch.tensor([c // ff if c < experts * ff else experts for c in range(inner)])
    limits = torch.where(lane_expert < experts, limit, shared_limit).double()
    g = torch.minimum(g64[:, :inner], limits)
    u = torch.maximum(torch.minimum(g64[:, inner:], limits), -limits)
    want = g * plain.sigmoid(1.702 * g) * (u + 1.0) * share.double().cpu()[:, lane_expert]
    close(act, want, dtype, "clamped lanes")
    assert float(g64[:, :inner].min()) < -limit         # the gate has no lower limit: such lanes are in the test


# ---- whole models -----------------------------------------------------------------------------------
LENGTHS = {"a": [1, 2, 23, 100, 131, 49], "b": [5, 19, 97, 201, 260, 100], "c": [3, 40, 130, 64, 1, 90],
           "d": [4, 31, 77, 150, 9, 60]}


@pytest.fixture(scope="module", params=sorted(TINY))
def model(request, tmp_path_factory):
    folder, cfg, page = make_folder(tmp_path_factory, request.param)
    requests = {f"r{i}": random_ids(n, cfg.vocab, 300 + i) for i, n in enumerate(LENGTHS[request.param])}
    return folder, cfg, page, requests, reference_logits(folder, requests)


def replay(folder, dtype, steps, max_tokens, page, max_requests=4, use_graphs=True):
    """What the replay program does, inside this process: every step through `Engine.step` on a pool of
    `max_tokens` tokens and `max_requests` slots; returns {step: logits}."""
    from tokenizer_b200.engine import Engine, StepEntry
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=-(-max_tokens // page), page_size=page,
                                max_requests=max_requests, use_graphs=use_graphs)
    live, out = {}, {}
    for record in steps:
        entries = []
        for item in record["entries"]:
            if item["id"] not in live:
                live[item["id"]] = engine.cache.open(item["id"])
            engine.cache.reserve(live[item["id"]], len(item["tokens"]))
            entries.append(StepEntry(live[item["id"]], item["tokens"], item.get("want", [])))
        logits = engine.step(entries)
        if logits.shape[0]:
            out[record["step"]] = logits.cpu().numpy()
        for name in record.get("end", []):
            engine.cache.close(live.pop(name))
        engine.cache.check()
    engine.check()
    return out


def compare(got, want, dtype, what):
    """float32: every logit within 1e-4.  bfloat16: per position, the root mean square of the difference (its
    mean over the vocabulary taken off) against that of the logits themselves: the operands' rounding (2^-9
    each) reaches the logits of these tiny models at about one part in a hundred, in a few positions several
    times that, while a key, a state, a kept input or an expert that is wrong moves a position's logits by
    their own size."""
    if dtype == "float32":
        return ru.compare(got, want, dtype, what)
    rel, where = [], []
    for name in sorted(got):
        for position in sorted(got[name]):
            row, ref = got[name][position], want[name][position]
            assert np.isfinite(row).all(), f"{what}: {name}[{position}] not finite"
            d, c = row - ref, ref - ref.mean()
            rel.append(float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((c ** 2).mean())))
            where.append((name, position))
    rel = np.array(rel)
    worst = int(rel.argmax())
    assert rel[worst] <= 0.25, f"{what} (bfloat16): request {where[worst][0]!r} position {where[worst][1]}: {rel[worst]:.3f}"
    assert np.percentile(rel, 90) <= 0.06, f"{what} (bfloat16): a tenth of the positions is off by {np.percentile(rel, 90):.3f} and more"


def test_every_layer_leaves_the_stream_the_plain_layers_leave(model):
    """The residual stream after every layer, float32."""
    from tokenizer_b200.engine import Engine, StepEntry
    folder, cfg, page, requests, _ = model
    ids = max(requests.values(), key=len)
    raw, w = plain.load_folder(folder)
    _, want = plain.forward(raw, w, ids, keep_layers=True)
    engine = Engine.from_folder(folder, dtype="float32", num_pages=-(-len(ids) // page) + 1, page_size=page,
                                max_requests=1, use_graphs=False)
    got = []
    for block in set(engine.model.blocks):
        def run(stream, ctx, cache, inner=block.forward):
            inner(stream, ctx, cache)
            got.append(stream.flush().clone())
        block.forward = run
    cache = engine.cache.open("r")
    engine.cache.reserve(cache, len(ids))
    engine.step([StepEntry(cache, ids, [0])])
    assert len(got) == len(want) == len(cfg.layers)
    for at, (a, b) in enumerate(zip(got, want)):
        err, size = float((a.cpu()[:len(ids)] - b.float()).abs().max()), float(b.abs().max())
        assert err <= 1e-4 * max(1.0, size), f"the stream after layer {at}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype):
    folder, cfg, page, requests, want = model
    steps = ru.steps_whole(requests)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    compare(got, want, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_token_by_token(model, dtype):
    """The last 40 tokens one by one: more than the chunks of 1, 7 and 24 positions, so that a chunk's edge passes
    under decoded tokens, and matrices and kept inputs are carried through every step."""
    folder, cfg, page, requests, want = model
    steps = ru.steps_decode_tail(requests, 40)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    compare(got, want, dtype, "decode tail")


def test_every_token_alone_from_the_first(model):
    """A sequence fed one token a step from its very first: the first tokens' kept inputs are the zeros before
    the start, and the first token sees itself and the sink."""
    folder, cfg, page, requests, want = model
    some = {k: v for k, v in requests.items() if len(v) <= 50}
    steps = ru.steps_portions(some, (1,))
    budget = max(ru.rounded64(len(v)) for v in some.values())
    got = ru.collect(steps, replay(folder, "float32", steps, budget, page))
    ru.compare(got, {k: want[k] for k in some}, "float32", "token by token from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 7, 3, 16, 2, 33, 5, 2, 64, 9), (2,), (31, 1, 1, 96)])
def test_portions(model, dtype, sizes):
    folder, cfg, page, requests, want = model
    if sizes == (2,):
        requests = {k: v for k, v in requests.items() if len(v) <= 100}
    steps = ru.steps_portions(requests, sizes)
    budget = max(ru.rounded64(len(v)) for v in requests.values())
    got = ru.collect(steps, replay(folder, dtype, steps, budget, page))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    compare(got, want, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [4, 2])
def test_mixed_batches_on_pages_and_slots_that_are_used_again(model, dtype, live):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=live, seed=live)
    assert peak < sum(ru.rounded64(len(v)) for v in requests.values()) and len(requests) > live
    got = ru.collect(steps, replay(folder, dtype, steps, peak, page, max_requests=live))
    assert {k: len(v) for k, v in got.items()} == {k: len(v) for k, v in requests.items()}
    compare(got, want, dtype, "mixed")


@pytest.mark.parametrize("kind", ["state_space", "attention"])
def test_models_of_one_kind_of_mixer_alone(kind, tmp_path_factory):
    """Layers of one kind only: a model that keeps no keys at all (every layer the recurrence: no page is ever
    read) and one that keeps no matrices, whole and in mixed batches on slots that are used again, float32."""
    from tiny_vizonex import attention, config, dense, mamba2, moe
    from tokenizer_b200 import write_random_model
    if kind == "state_space":
        cfg = config([mamba2(6, 12, 24, 3, 3, 2, dense(44)), mamba2(2, 36, 48, 1, 2, 4),
                      mamba2(4, 20, 8, 2, 4, 1, moe(5, 2, 12, 1.2, 1.7, shared=(20, 0.9)))],
                     vocab=210, width=72, eps=4e-6, taps=2)
    else:
        cfg = config([attention(5, 5, 12, 12, 0.7, size=33, mlp=dense(52)), attention(4, 1, 20, 28, 0.5, size=9),
                      attention(3, 1, 24, 8, 0.45, mlp=moe(6, 4, 10, 0.9, 1.3, groups=(2, 2)))],
                     vocab=190, width=60, eps=1e-5, taps=3)
    folder, page = str(tmp_path_factory.mktemp(f"vizonex_{kind}")), 16
    write_random_model(folder, cfg, 11, scale=SHARPEN)
    requests = {f"r{i}": random_ids(n, cfg.vocab, 500 + i) for i, n in enumerate([2, 70, 35, 141, 18, 66])}
    want = reference_logits(folder, requests)
    steps = ru.steps_whole(requests)
    got = ru.collect(steps, replay(folder, "float32", steps, max(ru.rounded64(len(v)) for v in requests.values()), page))
    ru.compare(got, want, "float32", f"{kind} alone, whole")
    steps, peak = ru.steps_mixed(requests, max_live=3, seed=5)
    got = ru.collect(steps, replay(folder, "float32", steps, peak, page, max_requests=3))
    ru.compare(got, want, "float32", f"{kind} alone, mixed")


def test_experts_chosen_token_by_token(tmp_path_factory):
    """With the router left as drawn, which experts a token uses changes from token to token (the other
    whole-model runs pin the choice, see `settle_routing`); in float32 a near tie is out of reach of rounding."""
    for name in ("a", "d"):
        folder, cfg, page = make_folder(tmp_path_factory, name, scale=dict(SHARPEN, **{r"\.router$": 20.0}), settled=False)
        requests = {f"r{i}": random_ids(n, cfg.vocab, 900 + i) for i, n in enumerate([70, 9, 131, 30, 2])}
        want = reference_logits(folder, requests)
        steps, peak = ru.steps_mixed(requests, max_live=3, seed=2)
        got = ru.collect(steps, replay(folder, "float32", steps, peak, page, max_requests=3))
        ru.compare(got, want, "float32", "experts chosen by the token")


def test_steps_launched_anew_agree_with_replayed_ones(model):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=3, seed=5)
    got = ru.collect(steps, replay(folder, "float32", steps, peak, page, max_requests=3, use_graphs=False))
    ru.compare(got, want, "float32", "without graphs")


def test_replay_program_drives_the_same_engine(model, tmp_path):
    folder, cfg, page, requests, want = model
    steps, peak = ru.steps_mixed(requests, max_live=3, seed=9)
    out = ru.run_trace(folder, "float32", steps, str(tmp_path), peak, page)
    ru.compare(ru.collect(steps, out), want, "float32", "the replay program")


# ---- generation ---------------------------------------------------------------------------------------
def near_best(cfg, w, prompt, tokens, dtype):
    logits = plain.forward(cfg, w, list(prompt) + list(tokens)).float()
    lead = logits[len(prompt) - 1:-1]
    chosen = lead.gather(1, torch.tensor(tokens)[:, None])[:, 0]
    slack = 1e-4 if dtype == "float32" else 0.1 * float(logits.abs().max())
    gap = lead.max(dim=1).values - chosen
    assert float(gap.max()) <= slack, f"token {int(gap.argmax())} lies {float(gap.max())} below the best logit"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(model, dtype):
    import tokenizer_b200 as tb
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine_model = tb.load_model(folder, dtype=dtype)
    for n in (1, 9, 70):
        prompt = random_ids(n, cfg.vocab, 500 + n)
        out = tb.generate(engine_model, prompt, tb.GenerateParams.greedy(24))
        assert out.reason == tb.StopReason.MAX_TOKENS and len(out.tokens) == 24
        near_best(raw, w, prompt, out.tokens, dtype)


def test_a_batch_through_the_scheduler_with_preemption_gives_each_request_its_own_ids(model):
    """Five prompts on a pool that cannot hold them all: requests are preempted and computed again, which for
    the recurrence and the convolutions means matrices and kept inputs that start from zero again."""
    import tokenizer_b200 as tb
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine_model = tb.load_model(folder, dtype="float32")
    prompts = [random_ids(n, cfg.vocab, 600 + n) for n in (30, 7, 55, 18, 41)]
    engine = tb.engine_for(engine_model, 192, page_size=page, max_requests=3, share_prefixes=False)
    results = tb.generate_batch(engine, prompts, tb.GenerateParams.greedy(20), max_batch_size=3, token_budget=48,
                                page_size=page)
    for prompt, result in zip(prompts, results):
        near_best(raw, w, prompt, result.tokens, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_on_the_device(model, dtype):
    """300 greedy steps without a visit to the host between them (captured and replayed): chunk edges pass under
    decoded tokens, pages behind them are given back, the states move on."""
    from tokenizer_b200.engine import Engine, StepEntry
    folder, cfg, page, requests, _ = model
    raw, w = plain.load_folder(folder)
    engine = Engine.from_folder(folder, dtype=dtype, num_pages=-(-2 * 384 // page), page_size=page, max_requests=2)
    prompts = [random_ids(5, cfg.vocab, 700), random_ids(41, cfg.vocab, 701)]
    caches, first = [], []
    for i, prompt in enumerate(prompts):
        c = engine.cache.open(i)
        engine.cache.reserve(c, len(prompt))
        first.append(int(engine.step([StepEntry(c, prompt, [len(prompt) - 1])]).argmax()))
        caches.append(c)
    history = engine.decode_steps([StepEntry(c, [t], [0]) for c, t in zip(caches, first)], 300)
    for i, prompt in enumerate(prompts):
        near_best(raw, w, prompt, [first[i]] + [step[i] for step in history], dtype)


def test_the_command_line_generates_from_a_configuration_of_this_design(tmp_path):
    """`--random-weights config.json` draws the weights the configuration declares; two prompts go through the
    scheduler and print ids that the plain implementation ranks best."""
    import json
    import os
    import subprocess
    import sys
    import tokenizer_b200 as tb
    cfg, seed, page = TINY["a"]()
    path = str(tmp_path / "config.json")
    with open(path, "w") as fh:
        json.dump(cfg.to_dict(), fh)
    folder = tb.write_random_model(str(tmp_path / "same"), cfg, 0)        # the command line's default seed
    raw, w = plain.load_folder(folder)
    prompts = [random_ids(11, cfg.vocab, 801), random_ids(40, cfg.vocab, 802)]
    cli = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "qwen-infer")
    args = [sys.executable, cli, "--random-weights", path, "--weights-seed", "0", "--dtype", "float32",
            "--max-tokens", "10", "--page-size", str(page)]
    for prompt in prompts:
        args += ["--ids", ",".join(str(t) for t in prompt)]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    lines = proc.stdout.strip().splitlines()
    assert len(lines) == 2
    for prompt, line in zip(prompts, lines):
        near_best(raw, w, prompt, [int(t) for t in line.split()], "float32")
