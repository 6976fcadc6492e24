"""Bosenex on the GPU against the plain implementation (tests/plain/bosenex_plain.py): each mechanism alone, then
whole models through the step function, the cache manager and the state slots in every cutting, then generation
through the engine."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import traces
from tests.bosenex_cases import CASES, assert_close_to_plain, make_model_dir, plain_logits, random_case, random_tokens
from tests.plain import bosenex_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64

LENGTHS = {"a": (70, 45, 128, 33, 2, 97), "b": (60, 9, 41, 3, 77), "c": (150, 66, 5, 90, 17, 2), "d": (90, 66, 5, 131, 40)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_dir(tmp_path_factory.mktemp(f"bx_{name}"), case) for name, case in CASES.items()}


def requests_for(name: str) -> dict[str, list[int]]:
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": random_tokens(300 + i, n, vocab) for i, n in enumerate(LENGTHS[name])}


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def tol_of(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def close(got, want, dtype, what=""):
    err = float((got.double().cpu() - want).abs().max())
    assert err <= tol_of(dtype) * max(1.0, float(want.abs().max())), (what, err)


# ---------------------------------------------------------------------------------------------
# each mechanism alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_projection_and_router(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(1)
    for rows, width, experts, top in ((37, 40, 5, 1), (9, 64, 8, 3), (130, 96, 3, 3), (4, 200, 33, 4)):
        h = torch.randn(rows, width, generator=gen).to(dtype)
        w = (torch.randn(experts, width, generator=gen) * 0.3).to(torch.bfloat16).float()
        b = torch.randn(experts, generator=gen)
        z = h.double() @ w.double().T + b.double()
        got = ops.small_linear(h.to(DEV), w.to(DEV), b.to(DEV))
        assert float((got.double().cpu() - z).abs().max()) < 1e-4
        dense, chosen, weight = ops.route_top_k(h.to(DEV), w.to(DEV), b.to(DEV), top)
        val, idx = torch.topk(z, top, dim=-1)
        assert torch.equal(chosen.cpu().long(), idx)
        assert float((weight.double().cpu() - torch.softmax(val, -1)).abs().max()) < 1e-5
        want = torch.zeros(rows, experts, dtype=F64).scatter_(1, idx, torch.softmax(val, -1))
        assert float((dense.double().cpu() - want).abs().max()) < 1e-5
        assert (dense.cpu() != 0).sum(1).eq(top).all()
    # equal logits: the lower index is chosen first
    h = torch.zeros(3, 16, dtype=dtype)
    dense, chosen, weight = ops.route_top_k(h.to(DEV), torch.zeros(6, 16, device=DEV), torch.tensor([0., 1., 1., 0., 1., 0.], device=DEV), 2)
    assert chosen.cpu().tolist() == [[1, 2]] * 3 and torch.allclose(weight.cpu(), torch.full((3, 2), 0.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_units(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(2)
    rows, experts, width, tail = 21, 3, 10, 7
    inner = experts * width + tail
    gu = (torch.randn(rows, 2 * inner, generator=gen) * 2).to(dtype)
    g, u = gu[:, :inner].double(), gu[:, inner:].double()
    close(ops.expert_act(gu.to(DEV), "relu"), torch.relu(g) * u, dtype, "relu")
    route = torch.rand(rows, experts, generator=gen)
    route[:, 1] = 0.0
    limit, tail_limit = 0.8, 1.7
    lim = torch.cat([torch.full((experts * width,), limit), torch.full((tail,), tail_limit)]).double()
    gg, uu = torch.minimum(g, lim), torch.maximum(torch.minimum(u, lim), -lim)
    weights = torch.cat([route.double().repeat_interleave(width, dim=1), torch.ones(rows, tail, dtype=F64)], dim=1)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1) * weights
    got = ops.expert_act(gu.to(DEV), "clamped_swish", limit, 1.702, 1.0, route=route.to(DEV), n_experts=experts, expert_width=width,
                         tail_limit=tail_limit)
    close(got, want, dtype, "experts")
    assert float(got[:, width: 2 * width].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_norms_and_join(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(3)
    rows, heads, dim, dims, base = 19, 5, 24, 12, 77.0
    buf = torch.randn(rows, heads * dim + 13, generator=gen).to(dtype)
    positions = torch.randint(0, 3000, (rows,), generator=gen)
    want = plain.rotate(buf[:, : heads * dim].double().view(rows, heads, dim), positions, dims, base).reshape(rows, -1)
    inv_freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).float()
    dev = buf.to(DEV)
    ops.rotate_half(dev, heads, dim, dims, inv_freq.to(DEV), positions.to(torch.int32).to(DEV))
    # the angle is a float32 product of a position in the thousands: its rounding is 1e-4 of a turn
    assert float((dev[:, : heads * dim].double().cpu() - want).abs().max()) <= (2e-3 if dtype == torch.float32 else 4e-2)
    assert torch.equal(dev[:, heads * dim:].cpu(), buf[:, heads * dim:]), "columns after the rotated heads changed"
    # groups of columns, each by its own root mean square, gate before or after
    groups, size, eps = 3, 20, 1e-3
    y = torch.randn(rows, groups * size, generator=gen) * 3
    gate = torch.randn(rows, groups * size, generator=gen).to(dtype)
    w = torch.randn(groups * size, generator=gen)
    z = gate.double()
    first = plain.rms((y.double() * z * torch.sigmoid(z)).view(rows, groups, size), eps).reshape(rows, -1) * w.double()
    after = plain.rms(y.double().view(rows, groups, size), eps).reshape(rows, -1) * w.double() * torch.sigmoid(z)
    close(ops.group_norm_gated(y.to(DEV), gate.to(DEV), w.to(DEV), groups, eps, True, dtype), first, dtype, "gate first")
    close(ops.group_norm_gated(y.to(DEV), gate.to(DEV), w.to(DEV), groups, eps, False, dtype), after, dtype, "gate after")
    x, a, b = (torch.randn(rows, 50, generator=gen) * s for s in (1.0, 5.0, 0.01))
    wa, wb = torch.randn(50, generator=gen), torch.randn(50, generator=gen)
    want = x.double() + 0.5 * (plain.rms_norm(a.double(), wa.double(), eps) + plain.rms_norm(b.double(), wb.double(), eps))
    got = ops.pair_norm_add(x.to(DEV), a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), eps, 0.5)
    assert float((got.double().cpu() - want).abs().max()) < 1e-5


def _entries(cuts, slots, fresh):
    starts = [0]
    for n in cuts:
        starts.append(starts[-1] + n)
    return i32(starts), i32(slots), i32(fresh)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 16, 16), (1, 64, 128), (3, 24, 40), (4, 8, 24), (1, 200, 8)])
def test_matrix_memory_recurrence_in_portions_and_slots(dtype, shape):
    """Two sequences side by side through state slots, cut into portions down to one row, in slots that held other
    sequences before; against the recurrence run whole."""
    from research_2_b200.kernels import ops

    heads, dim, vdim = shape
    gen = torch.Generator().manual_seed(4)
    cap, n_slots = 6.0, 3
    state = torch.full((n_slots, heads * ops.mlstm_state_floats(dim, vdim)), 123.0, device=DEV)   # what an earlier request left
    seqs = {}
    for name, n in (("x", 45), ("y", 23)):
        q, k = (torch.randn(n, heads * dim, generator=gen).to(dtype) for _ in range(2))
        v = torch.randn(n, heads * vdim, generator=gen).to(dtype)
        gates = torch.randn(n, 2 * heads, generator=gen) * 4
        gates[:, heads:] += 3
        log_i = plain.soft_cap(gates[:, :heads].double(), cap)
        log_f = torch.nn.functional.logsigmoid(plain.soft_cap(gates[:, heads:].double(), cap))
        want = plain.mlstm_cells(q.double().view(n, heads, dim) * dim ** -0.5, k.double().view(n, heads, dim),
                                 v.double().view(n, heads, vdim), log_i, log_f).reshape(n, -1)
        seqs[name] = (q, k, v, gates, want)
    plan = [[("x", 17), ("y", 1)], [("y", 2), ("x", 1)], [("x", 1)], [("y", 20), ("x", 26)]]
    slot, fed, got = {"x": 2, "y": 0}, {"x": 0, "y": 0}, {"x": [], "y": []}
    for step in plan:
        parts = [[seqs[name][i][fed[name]: fed[name] + n] for name, n in step] for i in range(4)]
        q, k, v, gates = (torch.cat(p).to(DEV) for p in parts)
        q_start, slots, fresh = _entries([n for _, n in step], [slot[name] for name, _ in step], [int(fed[name] == 0) for name, _ in step])
        out = ops.mlstm_scan(q, k, v, gates, cap, dim ** -0.5, state, q_start, slots, fresh, heads, dim, vdim).cpu()
        at = 0
        for name, n in step:
            got[name].append(out[at: at + n])
            at += n
            fed[name] += n
    for name in seqs:
        close(torch.cat(got[name]), seqs[name][4], dtype, f"{shape} {name}")
    assert float(state[1].min()) == 123.0, "a slot of no entry was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 16, 8, 1, 4), (4, 10, 12, 2, 3), (1, 40, 5, 1, 1), (3, 32, 24, 3, 2), (2, 64, 128, 1, 4)])
def test_state_space_recurrence_and_convolution_in_portions_and_slots(dtype, shape):
    from research_2_b200.kernels import ops

    heads, vdim, n_state, groups, taps = shape
    inner, bc = heads * vdim, groups * n_state
    channels = inner + 2 * bc
    gen = torch.Generator().manual_seed(5)
    conv = torch.randn(channels, taps, generator=gen) * 0.5
    conv_b, dt_bias, a_log, skip = (torch.randn(n, generator=gen) * 0.5 for n in (channels, heads, heads, heads))
    off = heads * n_state * vdim
    state = torch.full((4, off + (taps - 1) * channels), -55.0, device=DEV)
    seqs = {}
    for name, n in (("x", 39), ("y", 21)):
        xbc = torch.randn(n, channels, generator=gen).to(dtype)
        steps = torch.randn(n, heads, generator=gen)
        mixed = plain.causal_conv_silu(xbc.double(), conv.double(), conv_b.double())
        if dtype == torch.bfloat16:
            mixed = mixed.to(dtype).double()   # the convolution's output is stored in the activations' type
        want = plain.ssd_cells(mixed[:, :inner].view(n, heads, vdim), mixed[:, inner: inner + bc].view(n, groups, n_state),
                               mixed[:, inner + bc:].view(n, groups, n_state), torch.nn.functional.softplus(steps.double() + dt_bias.double()),
                               torch.exp(a_log.double()), skip.double()).reshape(n, -1)
        seqs[name] = (xbc, steps, want)
    plan = [[("x", 1)], [("x", 1), ("y", 2)], [("x", 2), ("y", 1)], [("y", 1), ("x", 20)], [("y", 17), ("x", 15)]]
    slot, fed, got = {"x": 3, "y": 1}, {"x": 0, "y": 0}, {"x": [], "y": []}
    for step in plan:
        xbc = torch.cat([seqs[name][0][fed[name]: fed[name] + n] for name, n in step]).to(DEV)
        steps = torch.cat([seqs[name][1][fed[name]: fed[name] + n] for name, n in step]).to(DEV)
        q_start, slots, fresh = _entries([n for _, n in step], [slot[name] for name, _ in step], [int(fed[name] == 0) for name, _ in step])
        row_entry = i32([e for e, (_, n) in enumerate(step) for _ in range(n)])
        mixed = ops.causal_conv(xbc, conv.to(DEV), conv_b.to(DEV), state, off, row_entry, q_start, slots, fresh)
        out = ops.ssd_scan(mixed[:, :inner], mixed[:, inner: inner + bc], mixed[:, inner + bc:], steps, dt_bias.to(DEV), a_log.to(DEV),
                           skip.to(DEV), state, q_start, slots, fresh, heads, groups, n_state, vdim, conv_in=xbc, conv_taps=taps,
                           conv_state_off=off).cpu()
        at = 0
        for name, n in step:
            got[name].append(out[at: at + n])
            at += n
            fed[name] += n
    for name in seqs:
        close(torch.cat(got[name]), seqs[name][2], dtype, f"{shape} {name}")
    assert float(state[0].max()) == -55.0 and float(state[2].max()) == -55.0, "a slot of no entry was written"


def _attention_case(dtype, heads, kv, dim, vdim, window, softcap, page, lengths, new_rows, seed, plant=None):
    """Entries of `lengths` keys each whose last `new_rows` positions are this step's rows: the older keys and values are
    put into a paged cache whose pages lie in a scrambled order, then one mixed batch runs. `plant` = (entry, row,
    distance): the key `distance` positions before that row is made to stand out (its score dwarfs the others) and its
    value is made large, so that seeing or not seeing it decides the output. -> (outputs per entry, the plain ones)."""
    from research_2_b200.cache.arena import KVArena, MemberSpec, derive_groups
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(seed)
    member = MemberSpec(kv, dim, window, vdim, 0)
    n_pages = sum(-(-n // page) for n in lengths) + 3
    groups, index = derive_groups([member], page, n_pages)
    arena = KVArena([member], groups, index, dtype, DEV)
    arena.fill_(77.0)
    cache = arena.members[0]
    order = torch.randperm(n_pages, generator=gen).tolist()
    tables = torch.zeros(len(lengths), max(-(-n // page) for n in lengths) + 1, dtype=torch.int32)
    sinks = torch.randn(heads, generator=gen)
    scale = 0.3
    qs, ks, vs, gs, slots, row_entry, positions, q_start = [], [], [], [], [], [], [], [0]
    for e, n in enumerate(lengths):
        q, k = torch.randn(n, heads, dim, generator=gen), torch.randn(n, kv, dim, generator=gen)
        v, g = torch.randn(n, kv, vdim, generator=gen), torch.randn(n, heads, generator=gen)
        if plant is not None and plant[0] == e:
            row, j = n - new_rows[e] + plant[1], n - new_rows[e] + plant[1] - plant[2]
            if j >= 0:
                k[j] = q[row, 0] * 8.0
                v[j] = 40.0
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        qs.append(q), ks.append(k), vs.append(v), gs.append(g)
        for i in range(-(-n // page)):
            tables[e, i] = order.pop() + 1
        slot = [int(tables[e, j // page]) * page + j % page for j in range(n)]
        first_new = n - new_rows[e]
        if window > 0:   # pages that lie wholly before the window of the entry's first new row have been given back
            for i in range(max(0, first_new - window + 1) // page):
                tables[e, i] = 0
        if first_new:
            ops.kv_write(k[:first_new].reshape(first_new, -1).to(dtype).to(DEV), v[:first_new].reshape(first_new, -1).to(dtype).to(DEV),
                         cache.k, cache.v, i32(slot[:first_new]), kv, dim, page, cache.page_stride, cache.n_pages, v_head_dim=vdim)
        slots += slot[first_new:]
        row_entry += [e] * new_rows[e]
        positions += list(range(first_new, n))
        q_start.append(q_start[-1] + new_rows[e])
    new = lambda parts: torch.cat([p[len(p) - r:].reshape(r, -1) for p, r in zip(parts, new_rows)])  # noqa: E731
    q_new, k_new, v_new = (new(p).to(dtype).to(DEV) for p in (qs, ks, vs))
    g_new = new(gs).to(DEV)
    ops.kv_write(k_new, v_new, cache.k, cache.v, i32(slots), kv, dim, page, cache.page_stride, cache.n_pages, v_head_dim=vdim)
    out = ops.paged_attention(
        q_new, cache.k, cache.v, cache.page_stride, page, cache.n_pages, tables.to(DEV), i32(row_entry), i32(positions), i32(lengths),
        heads, kv, dim, scale, window, decode_only=all(r == 1 for r in new_rows), max_context=max(lengths), q_start=i32(q_start),
        n_tiles=sum(-(-r // 64) for r in new_rows), v_head_dim=vdim, softcap=softcap, sinks=sinks.to(DEV), head_gate=g_new).float().cpu()
    got, want, at = [], [], 0
    for e, n in enumerate(lengths):
        r = new_rows[e]
        core = plain.attention_core(qs[e][n - r:].double(), ks[e].double(), vs[e].double(), scale, softcap, window or None,
                                    sinks.double(), first_row=n - r)
        want.append((core * torch.sigmoid(gs[e][n - r:].double())[:, :, None]).reshape(r, -1))
        got.append(out[at: at + r].double())
        at += r
    return got, want


ATTENTION_SHAPES = [
    # heads, kv heads, dim, vdim, window, softcap, page
    (4, 2, 32, 32, 44, 20.0, 16), (8, 1, 64, 64, 70, 0.0, 32), (2, 2, 16, 16, 5, 3.0, 8), (3, 1, 24, 40, 9, 0.0, 4),
    (2, 1, 128, 64, 130, 50.0, 16), (6, 2, 96, 16, 0, 30.0, 8), (5, 5, 48, 48, 1, 0.0, 16), (6, 3, 96, 96, 120, 30.0, 16),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_attention_prompts_portions_and_decoded_rows(dtype, shape):
    for lengths, new_rows in (((150, 37, 201, 64, 9), (150, 2, 77, 1, 9)), ((300, 1, 45, 130), (1, 1, 1, 1)), ((700, 333, 64), (700, 1, 3))):
        got, want = _attention_case(dtype, *shape, lengths, new_rows, seed=7)
        for e, (a, b) in enumerate(zip(got, want)):
            close(a, b, dtype, f"{shape} {lengths} entry {e}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_that_stands_out_at_every_edge(dtype, decode):
    """One key whose score dwarfs all others and whose value is 40: at the last place inside the window the row's first
    head returns (nearly) that value, one place further out an ordinary mixture; for rows in a prompt's portion and for
    decoded rows, with the key behind a page's border; without a window a key 600 places back among hundreds."""
    heads, kv, dim, page, n = 2, 1, 32, 16, 230
    for window, row_pos, distance, seen in (
        (36, n - 1, 35, True), (36, n - 1, 36, False), (36, n - 1, 0, True), (36, n - 1, 1, True), (36, 100, 35, True),
        (36, 100, 36, False), (16, 127, 15, True), (16, 127, 16, False), (16, 128, 15, True), (16, 128, 16, False),
        (1, 77, 0, True), (1, 77, 1, False), (0, n - 1, n - 1, True), (0, 100, 100, True),
    ):
        if decode:
            lengths, new_rows, row = (row_pos + 1, 50), (1, 1), 0
        else:
            lengths, new_rows, row = (n, 50), (n - 60, 2), row_pos - 60
        got, want = _attention_case(dtype, heads, kv, dim, dim, window, 0.0, page, lengths, new_rows, seed=11, plant=(0, row, distance))
        a, b = got[0][row], want[0][row]
        close(a, b, dtype, f"window {window} row {row_pos} distance {distance}")
        assert (float(b[:dim].abs().max()) > 4.0) == seen, (window, row_pos, distance, float(b[:dim].abs().max()))
        assert (float(a[:dim].abs().max()) > 4.0) == seen, (window, row_pos, distance, decode, float(a[:dim].abs().max()))
    got, want = _attention_case(dtype, heads, kv, dim, dim, 0, 25.0, page, (700, 650), (1, 40), seed=12, plant=(0, 0, 600))
    close(got[0][0], want[0][0], dtype, "a far key")
    assert float(want[0][0][:dim].abs().max()) > 4.0 and float(got[0][0][:dim].abs().max()) > 4.0


# ---------------------------------------------------------------------------------------------
# whole models in every cutting


def cut(requests, mode: str) -> traces.TraceBuilder:
    if mode == "whole":
        return traces.whole(requests)
    if mode == "decode":
        return traces.prefill_then_decode(requests, 48)
    if mode == "portions":
        return traces.portions(requests)
    if mode == "tiny_portions":
        return traces.portions(requests, sizes=(2, 3, 2, 5, 2, 2, 9))
    return traces.mixed(requests, max_live=4)


def run_trace(folder, tb, dtype, page_size, max_tokens=None, max_seq_len=0):
    """Replays the trace in a pool of the trace's own peak demand plus one page (or `max_tokens`), cache and state slots
    filled with loud values first. -> ({step: logits}, how many pages had two owners or more, the replay)."""
    from research_2_b200.engine.replay import Replay

    live, round_to = traces.max_live(tb), 64
    if max_tokens is None:
        max_tokens, round_to = (traces.peak_pages(tb, page_size) + 1) * page_size, page_size
    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size, max_live=max(live, 1), round_to=round_to, max_seq_len=max_seq_len)
    replay.step_fn.arena.fill_(64.0)
    for t in replay.step_fn.state_tensors:
        t.fill_(-9.0)
    owners: dict[tuple[int, int], set] = {}
    out = {}
    for record in tb.steps:
        logits = replay.step(record)
        if logits is not None:
            out[record["step"]] = logits
        for rid, per_group in replay.pages_of_last_step.items():
            for g, pages in enumerate(per_group):
                for page in pages:
                    owners.setdefault((g, page), set()).add(rid)
    assert replay.cache.check() == ""
    for g in range(len(replay.cache.groups)):
        assert replay.cache.n_free(g) == replay.cache.groups[g].num_pages, "pages were lost"
    return out, sum(len(v) >= 2 for v in owners.values()), replay


def compare(folder, requests, tb, outputs, dtype, what):
    assert sorted(outputs) == sorted(tb.rows)
    per_request: dict[str, dict[int, np.ndarray]] = {}
    for step, rows in tb.rows.items():
        for (rid, pos), logits in zip(rows, outputs[step]):
            assert pos not in per_request.setdefault(rid, {}), f"{what}: position {pos} of {rid} written twice"
            per_request[rid][pos] = logits
    for rid, ids in requests.items():
        assert sorted(per_request[rid]) == list(range(len(ids))), f"{what}: request {rid} misses positions"
        got = np.stack([per_request[rid][p] for p in range(len(ids))])
        assert_close_to_plain(got, folder, ids, dtype, what=f"{what} request {rid}")
    return per_request


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("mode", ["whole", "decode", "portions", "tiny_portions", "mixed"])
def test_cuttings(folders, name, dtype, mode):
    folder, requests = folders[name], requests_for(name)
    if mode == "tiny_portions":
        requests = dict(list(requests.items())[:3])
    tb = cut(requests, mode)
    outputs, reused, replay = run_trace(folder, tb, dtype, CASES[name]["page_size"])
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")
    if mode == "mixed":
        assert traces.max_live(tb) == 4 and len(requests) > 4, "state slots are used again"
        if replay.model.cache_members:
            assert reused >= 4, f"only {reused} pages passed from one request to another"


@pytest.mark.parametrize("seed", range(100, 108))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layers in any order and sizes of any kind: float32 within its floor in three cuttings, bfloat16 within its own
    (positions at which the design is discontinuous excused)."""
    case = random_case(seed)
    folder = make_model_dir(tmp_path / "model", case)
    ids = random_tokens(seed, case["length"], case["config"]["vocab"])
    requests = {"x": ids, "y": ids[: max(3, len(ids) // 3)], "z": ids[5:]}
    for dtype, modes in (("float32", ("whole", "portions", "mixed")), ("bfloat16", ("mixed",))):
        for mode in modes:
            tb = cut(requests, mode) if mode != "mixed" else traces.mixed(requests, max_live=2)
            outputs, _, _ = run_trace(folder, tb, dtype, case["page_size"])
            compare(folder, requests, tb, outputs, dtype, f"seed {seed} {dtype} {mode}")


def test_float32_logits_do_not_depend_on_the_cutting_at_all(folders):
    for name in ("a", "b", "c"):
        folder, requests = folders[name], requests_for(name)
        results = {}
        for mode in ("whole", "decode", "portions", "mixed"):
            tb = cut(requests, mode)
            results[mode] = compare(folder, requests, tb, run_trace(folder, tb, "float32", CASES[name]["page_size"])[0], "float32", f"{name}/{mode}")
        for mode in ("decode", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                for pos, logits in rows.items():
                    assert np.array_equal(logits, results[mode][rid][pos]), f"{name}: {mode} differs from whole at {rid}[{pos}]"


def test_long_decoding_through_a_small_pool(folders):
    """400 tokens, 390 of them decoded one by one: the windows pass over decoded tokens, the window groups give their
    pages back (8 pages a group hold it all), the states are carried 390 times."""
    name = "a"
    folder, page = folders[name], CASES[name]["page_size"]
    ids = random_tokens(21, 400, CASES[name]["config"]["vocab"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=390)
    for dtype in ("float32", "bfloat16"):
        outputs, _, replay = run_trace(folder, tb, dtype, page, max_tokens=8 * page, max_seq_len=512)
        compare(folder, {"x": ids}, tb, outputs, dtype, f"long decoding in a small pool {dtype}")
        assert sorted(g.window for g in replay.cache.groups) == [7, 24]


def test_first_tokens(folders):
    for name in ("a", "b", "c"):
        folder = folders[name]
        ids = random_tokens(7, 5, CASES[name]["config"]["vocab"])
        tb = traces.TraceBuilder()
        tb.step([("x", ids[:1], [0])])
        tb.step([("x", ids[1:2], [0])])
        tb.step([("x", ids[2:4], [0, 1])])
        tb.step([("x", ids[4:5], [0])], end=["x"])
        for dtype in ("float32", "bfloat16"):
            compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, CASES[name]["page_size"], max_tokens=64)[0], dtype, f"first tokens {name} {dtype}")


def test_trace_run_program(folders, tmp_path):
    folder, name = folders["d"], "d"
    requests = {k: v for k, v in list(requests_for(name).items())[:3]}
    tb = traces.mixed(requests, max_live=3)
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in tb.steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "bfloat16",
         "--out", str(out), "--max-tokens", str(sum(-(-len(v) // 64) * 64 for v in requests.values()))],
        input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(len(tb.steps))]
    vocab = CASES[name]["config"]["vocab"]
    outputs = {int(p.stem): np.fromfile(p, dtype="<f4").reshape(-1, vocab) for p in out.glob("*.f32")}
    compare(folder, requests, tb, outputs, "bfloat16", "trace_run program")


# ---------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler


def test_greedy_generation_through_the_engine(folders):
    """Prompts of unequal length through `generate` (scheduler, portions under a small token budget, state slots, CUDA
    graphs): float32 tokens equal the plain implementation's; bfloat16 tokens are (nearly) the best by the plain
    logits of the sequence so far."""
    import research_2_b200

    for name in ("a", "c"):
        folder, vocab = folders[name], CASES[name]["config"]["vocab"]
        prompts = [random_tokens(40 + i, n, vocab) for i, n in enumerate((5, 61, 18, 33))]
        cfg, w = plain.read_model(folder)
        want = [plain.generate(cfg, w, p, 10) for p in prompts]
        got = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="float32", device=DEV, block_size=8,
                                       max_batch_tokens=32, max_requests=3, max_seq_len=128)
        assert got == want, (name, got, want)
        got16 = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="bfloat16", device=DEV, block_size=16,
                                         max_batch_tokens=48, max_requests=4, max_seq_len=128)
        for prompt, tokens in zip(prompts, got16):
            assert len(tokens) == 10
            logits = plain_logits(folder, (prompt + tokens)[:-1])
            slack = 2 * 3e-2 * float(np.abs(logits).max())
            for i, tok in enumerate(tokens):
                row = logits[len(prompt) - 1 + i]
                assert float(row[tok]) >= float(row.max()) - slack, (name, i, tok)


def test_generation_in_a_pool_that_forces_preemption(folders):
    """A preempted request is computed again from its first token: its state slot starts from zero."""
    import research_2_b200

    name = "d"
    folder, vocab = folders[name], CASES[name]["config"]["vocab"]
    prompts = [random_tokens(60 + i, n, vocab) for i, n in enumerate((30, 44, 25))]
    cfg, w = plain.read_model(folder)
    want = [plain.generate(cfg, w, p, 10) for p in prompts]
    got = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="float32", device=DEV, block_size=4,
                                   max_batch_tokens=16, max_requests=3, max_seq_len=64, num_slabs=30)
    assert got == want, (got, want)


def test_command_line(folders):
    folder = folders["b"]
    proc = subprocess.run([sys.executable, "-m", "research_2_b200", "generate", "--model", str(folder), "--prompt-tokens", "5,17,3",
                           "--max-new-tokens", "4", "--dtype", "float32", "--max-seq-len", "64"],
                          capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout.strip().splitlines()[-1])["tokens"]
    cfg, w = plain.read_model(folder)
    assert tokens == plain.generate(cfg, w, [5, 17, 3], 4)
