"""Zirunex on the GPU against the plain implementation (tests/plain/zirunex_plain.py): each mechanism
alone, then whole models through the step function and the cache manager in every cutting, then
generation through the engine."""

from __future__ import annotations

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import zirunex_plain as plain
from tests.zirunex_cases import CASES, assert_close_to_plain, make_model_dir, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"

LENGTHS = {"a": (70, 45, 128, 33, 2, 97), "b": (60, 9, 41, 3, 77), "c": (300, 130, 64, 200, 17, 2, 129), "d": (150, 66, 5, 131, 40, 90)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_dir(tmp_path_factory.mktemp(f"zx_{name}"), case) for name, case in CASES.items()}


def requests_for(name: str) -> dict[str, list[int]]:
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": random_tokens(300 + i, n, vocab) for i, n in enumerate(LENGTHS[name])}


# ---------------------------------------------------------------------------------------------
# each mechanism alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_norm_and_head_norm(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(1)
    for width, unit in ((40, True), (256, False), (1000, True)):
        x = torch.randn(7, width, generator=gen) * 3.0
        w = torch.randn(width, generator=gen) * 0.3
        rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32)
        want = plain.stream_norm(x.double(), w.double(), 1e-5) if unit else plain.head_norm(x.double(), w.double(), 1e-5)
        got = ops.rms_norm(x.to(DEV), w.to(DEV), 1e-5, dtype, unit_offset=unit)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(got.cpu().double(), want, atol=tol * float(want.abs().max()), rtol=0)
        picked = ops.rms_norm(x.to(DEV), w.to(DEV), 1e-5, dtype, rows=rows.to(DEV), unit_offset=unit)
        assert torch.equal(picked.cpu(), got.cpu()[rows.long()])
    # the heads of a stacked projection: query heads with one gain, key heads with another, the rest untouched
    n_q, n_k, d, extra = 3, 2, 24, 50
    buf = (torch.randn(6, (n_q + n_k) * d + extra, generator=gen) * 2.0).to(dtype)
    gq, gk = torch.rand(d, generator=gen) + 0.5, torch.rand(d, generator=gen) + 0.5
    ref = buf.double().clone()
    heads = ref[:, : (n_q + n_k) * d].view(6, n_q + n_k, d)
    ref[:, : n_q * d] = plain.head_norm(heads[:, :n_q], gq.double(), 1e-6).reshape(6, -1)
    ref[:, n_q * d: (n_q + n_k) * d] = plain.head_norm(heads[:, n_q:], gk.double(), 1e-6).reshape(6, -1)
    dev = buf.to(DEV)
    ops.head_norm(dev, n_q, n_k, d, gq.to(DEV), gk.to(DEV), 1e-6)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(dev.cpu().double(), ref, atol=tol * float(ref.abs().max()), rtol=0)
    assert torch.equal(dev.cpu()[:, (n_q + n_k) * d:], buf[:, (n_q + n_k) * d:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(5, 2, 48, 16, 8), (4, 4, 64, 64, 16), (3, 1, 24, 40, 4), (2, 1, 256, 128, 2)])
def test_head_norm_that_writes_the_cache(dtype, sizes):
    """The launch that norms the query and key heads also puts the normed keys and the values into the rows'
    slots: the cache then holds exactly what the projection's key columns hold, and the value columns."""
    from research_2_b200.cache.arena import KVArena, MemberSpec, derive_groups
    from research_2_b200.kernels import ops

    n_q, n_k, d, vd, page = sizes
    rows, extra = 37, 24
    gen = torch.Generator().manual_seed(3)
    width = (n_q + n_k) * d + n_k * vd + extra
    buf = (torch.randn(rows, width, generator=gen) * 2.0).to(dtype)
    gq, gk = torch.rand(d, generator=gen) + 0.5, torch.rand(d, generator=gen) + 0.5
    member = MemberSpec(n_k, d, 0, vd, 0)
    groups, index = derive_groups([member], page, 40)
    arena = KVArena([member], groups, index, dtype, DEV)
    arena.fill_(9.0)
    cache = arena.members[0]
    slots = (torch.randperm(40 * page, generator=gen)[:rows] + page).to(torch.int32)
    dev = buf.to(DEV)
    slots_dev = slots.to(DEV)   # (the scatter description holds its address only)
    scatter = ops.kv_scatter(slots_dev, cache.k, cache.v, cache.page_stride, page, cache.n_pages, (n_q + n_k) * d, n_k * vd, vd)
    ops.head_norm(dev, n_q, n_k, d, gq.to(DEV), gk.to(DEV), 1e-6, kv=scatter)
    got = dev.cpu()
    heads = buf.double()[:, : (n_q + n_k) * d].view(rows, n_q + n_k, d)
    want_q = plain.head_norm(heads[:, :n_q], gq.double(), 1e-6).reshape(rows, -1)
    want_k = plain.head_norm(heads[:, n_q:], gk.double(), 1e-6).reshape(rows, -1)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(got[:, : n_q * d].double(), want_q, atol=tol * float(want_q.abs().max()), rtol=0)
    assert torch.allclose(got[:, n_q * d: (n_q + n_k) * d].double(), want_k, atol=tol * float(want_k.abs().max()), rtol=0)
    assert torch.equal(got[:, (n_q + n_k) * d:], buf[:, (n_q + n_k) * d:]), "values and what follows are left alone"
    pool = arena.tensors[0].cpu()
    k_elems = n_k * page * d
    for r in range(rows):
        pg, off = int(slots[r]) // page, int(slots[r]) % page
        k_page = pool[pg, :k_elems].view(n_k, page, d)
        v_page = pool[pg, k_elems: k_elems + n_k * page * vd].view(n_k, page, vd)
        assert torch.equal(k_page[:, off], got[r, n_q * d: (n_q + n_k) * d].view(n_k, d)), r
        assert torch.equal(v_page[:, off], buf[r, (n_q + n_k) * d: (n_q + n_k) * d + n_k * vd].view(n_k, vd)), r
    written = torch.zeros(41, page, dtype=torch.bool)
    written[slots.long() // page, slots.long() % page] = True
    untouched = pool[:, :k_elems].view(41, n_k, page, d)[~written[:, None, :].expand(41, n_k, page)]
    assert bool((untouched == 9.0).all()), "a slot of no row was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_unit_and_scaled_embedding(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(2)
    for inner, limit in ((24, 0.4), (1500, 2.0)):
        gu = (torch.randn(5, 2 * inner, generator=gen) * 3.0).to(dtype)   # most values beyond the clamp
        want = plain.gated_unit(gu[:, :inner].double(), gu[:, inner:].double(), limit)
        got = ops.gated_act(gu.to(DEV), limit, 1.702, 1.0).cpu().double()
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        assert torch.allclose(got, want, atol=tol * float(want.abs().max()), rtol=0)
    table = torch.randn(30, 72, generator=gen).to(dtype)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    got = ops.embed(ids.to(DEV), table.to(DEV), scale=2.5).cpu()
    assert torch.allclose(got.double(), plain.embed(ids, table.double(), 2.5), atol=1e-6, rtol=0)


def _attention_case(dtype, n_heads, n_kv, dim, vdim, window, keep, page, lengths, new_rows, seed, plant=None):
    """Entries of `lengths` keys each whose last `new_rows` positions are this step's rows: the older keys
    and values are put into a paged cache (pages in a scrambled order), then one mixed batch runs. Returns
    (the kernel's output per entry, the plain implementation's). `plant` = (entry, row, distance): the key
    `distance` positions before that row is made to stand out (its score dwarfs the others) and its value
    is made large, so that seeing or not seeing it decides the output."""
    from research_2_b200.cache.arena import KVArena, MemberSpec, derive_groups
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(seed)
    member = MemberSpec(n_kv, dim, window, vdim, keep)
    n_pages = sum(-(-n // page) for n in lengths) + 3
    groups, index = derive_groups([member], page, n_pages)
    arena = KVArena([member], groups, index, dtype, DEV)
    arena.fill_(77.0)
    cache = arena.members[0]
    order = torch.randperm(n_pages, generator=gen).tolist()
    width = max(-(-n // page) for n in lengths) + 1
    tables = torch.zeros(len(lengths), width, dtype=torch.int32)
    qs, ks, vs, gs, slots, row_entry, positions, q_start = [], [], [], [], [], [], [], [0]
    for e, n in enumerate(lengths):
        q = torch.randn(n, n_heads, dim, generator=gen)
        k = torch.randn(n, n_kv, dim, generator=gen)
        v = torch.randn(n, n_kv, vdim, generator=gen)
        g = torch.randn(n, n_heads * vdim, generator=gen)
        if plant is not None and plant[0] == e:
            row, distance = n - new_rows[e] + plant[1], plant[2]
            j = row - distance
            if j >= 0:
                k[j] = q[row, 0] * 8.0      # its score with the row's first head dwarfs every other
                v[j] = 40.0
        q, k, v, g = (t.to(dtype).float() for t in (q, k, v, g))
        qs.append(q), ks.append(k), vs.append(v), gs.append(g)
        for i in range(-(-n // page)):
            tables[e, i] = order.pop() + 1
        slot = [int(tables[e, j // page]) * page + j % page for j in range(n)]
        first_new = n - new_rows[e]
        # the cache manager of a window group has given back the pages that lie wholly before the window of
        # the entry's first new row (and after the kept first tokens): they read as the null page here too
        if window > 0:
            first_needed = max(0, first_new - window + 1) // page
            for i in range(-(-keep // page) if keep else 0, first_needed):
                tables[e, i] = 0
        old = torch.tensor(slot[:first_new], dtype=torch.int32)
        if len(old):
            ops.kv_write(k[:first_new].reshape(first_new, -1).to(dtype).to(DEV), v[:first_new].reshape(first_new, -1).to(dtype).to(DEV),
                         cache.k, cache.v, old.to(DEV), n_kv, dim, page, cache.page_stride, cache.n_pages, v_head_dim=vdim)
        slots += slot[first_new:]
        row_entry += [e] * new_rows[e]
        positions += list(range(first_new, n))
        q_start.append(q_start[-1] + new_rows[e])
    new = lambda parts: torch.cat([p[len(p) - r:].reshape(r, -1) for p, r in zip(parts, new_rows)]).to(dtype).to(DEV)  # noqa: E731
    i32 = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)  # noqa: E731
    q_new, k_new, v_new, g_new = new(qs), new(ks), new(vs), new(gs)
    decode_only = all(r == 1 for r in new_rows)
    fused = None
    if decode_only and dtype == torch.bfloat16 and vdim == dim:
        fused = ops.decode_attention_fused(
            q_new, k_new, v_new, i32(slots), cache.k, cache.v, cache.page_stride, page, cache.n_pages, tables.to(DEV),
            i32(row_entry), i32(positions), i32(lengths), n_heads, n_kv, dim, 0.3, window, max(lengths), keep_first=keep,
            sink=True, gate=g_new, exact_weights=True)
    if fused is None:
        ops.kv_write(k_new, v_new, cache.k, cache.v, i32(slots), n_kv, dim, page, cache.page_stride, cache.n_pages, v_head_dim=vdim)
        n_tiles = sum(-(-r // 64) for r in new_rows)
        fused = ops.paged_attention(
            q_new, cache.k, cache.v, cache.page_stride, page, cache.n_pages, tables.to(DEV), i32(row_entry), i32(positions),
            i32(lengths), n_heads, n_kv, dim, 0.3, window, decode_only=decode_only, max_context=max(lengths),
            q_start=i32(q_start), n_tiles=n_tiles, v_head_dim=vdim, keep_first=keep, sink=True, gate=g_new)
    got = fused.float().cpu()
    out, want, at = [], [], 0
    for e, n in enumerate(lengths):
        r = new_rows[e]
        heads = plain.attention_heads(qs[e][n - r:].double(), ks[e].double(), vs[e].double(), 0.3,
                                      window if window > 0 else 10 ** 9, keep, first_position=n - r)
        want.append(heads.reshape(r, -1) * torch.sigmoid(gs[e][n - r:].double()))
        out.append(got[at: at + r].double())
        at += r
    return out, want


ATTENTION_SHAPES = [
    # heads, kv heads, dim, vdim, window, kept, page
    (4, 2, 32, 32, 44, 7, 16),
    (8, 1, 64, 64, 70, 70, 32),
    (2, 2, 16, 16, 5, 0, 8),
    (3, 1, 24, 40, 9, 12, 4),      # only the general kernel takes it
    (2, 1, 128, 128, 130, 3, 16),
    (6, 2, 32, 32, 20, 2, 8),      # three query heads a kv head
    (5, 5, 48, 48, 33, 1, 16),
    (6, 2, 64, 64, 50, 3, 16),     # the same at the tcgen05 kernel's head size
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_attention_prompts_portions_and_decoded_rows(dtype, shape):
    """Whole prompts, portions that start in the middle of a window and of a page, and single decoded rows
    in one batch; then a batch of decoded rows only (the kernel that writes the cache itself)."""
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for lengths, new_rows in (((150, 37, 201, 64, 9), (150, 2, 77, 1, 9)), ((300, 1, 45, 130), (1, 1, 1, 1))):
        out, want = _attention_case(dtype, *shape, lengths, new_rows, seed=7)
        for e, (a, b) in enumerate(zip(out, want)):
            err = (a - b).abs().max(dim=1).values
            assert float(err.max()) <= tol * max(1.0, float(b.abs().max())), (shape, lengths, e, int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dim", [32, 64])
def test_one_key_that_stands_out_at_every_edge(dtype, decode, dim):
    """One key whose score dwarfs all others and whose value is 40: at the last place inside the window
    the row's first head returns (nearly) that value, one place further out it returns an ordinary
    mixture; the same at the last kept first token and the first one that is not kept; for rows in a
    prompt's portion and for decoded rows, with the key far behind a page's border."""
    heads, kv, window, keep, page = 2, 1, 36, 5, 16   # (head size 64 in bfloat16: the tcgen05 kernel)
    n = 230
    for row_pos, distance, seen in (
        (n - 1, window - 1, True), (n - 1, window, False),              # the window's far edge
        (n - 1, n - 1 - (keep - 1), True), (n - 1, n - 1 - keep, False),  # the last kept token and the next one
        (n - 1, 0, True), (n - 1, 1, True), (n - 1, n - 1, True),       # itself, its neighbour, the very first token
        (100, window - 1, True), (100, window, False), (100, 100 - (keep - 1), True), (100, 100 - keep, False),
    ):
        if decode:
            lengths, new_rows, row = (row_pos + 1, 50), (1, 1), 0
        else:
            lengths, new_rows, row = (n, 50), (n - 60, 2), row_pos - 60
            if row < 0:
                continue
        out, want = _attention_case(dtype, heads, kv, dim, dim, window, keep, page, lengths, new_rows, seed=11,
                                    plant=(0, row, distance))
        a, b = out[0][row], want[0][row]
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), (row_pos, distance, decode)
        # the plain implementation itself shows the planted key exactly where the mask says
        assert (float(b[:dim].abs().max()) > 5.0) == seen, (row_pos, distance, float(b[:dim].abs().max()))
        assert (float(a[:dim].abs().max()) > 5.0) == seen, (row_pos, distance, decode, float(a[:dim].abs().max()))


@pytest.mark.parametrize("page", [8, 16, 32, 64])
def test_head_size_64_on_both_prefill_kernels(page):
    """Head size 64 runs on the tcgen05 kernel (two-term weights in the two halves of a score buffer, kept
    tiles before the window's, sink, gate) and, switched off, on the mma.sync kernel: both against the plain
    implementation, with one prompt (CTA pairs share the keys), several, and decoded rows beside portions."""
    from research_2_b200.kernels import ops

    for tc in (True, False):
        before_setting = ops.use_prefill_tc_extras(tc)
        before = ops.kernel_uses()
        try:
            for shape in ((4, 2, 64, 64, 100, 70, page), (8, 1, 64, 64, 70, 5, page), (2, 2, 64, 64, 1000, 0, page)):
                for lengths, new_rows in (((700,), (700,)), ((150, 37, 401, 64, 9), (150, 2, 277, 1, 9)), ((520, 300), (200, 129))):
                    out, want = _attention_case(torch.bfloat16, *shape, lengths, new_rows, seed=5)
                    for e, (a, b) in enumerate(zip(out, want)):
                        err = (a - b).abs().max(dim=1).values
                        assert float(err.max()) <= 2e-2 * max(1.0, float(b.abs().max())), (tc, shape, lengths, e, int(err.argmax()), float(err.max()))
        finally:
            ops.use_prefill_tc_extras(before_setting)
        after = ops.kernel_uses()
        name = "attention_prefill_tc" if tc else "attention_prefill"
        assert after.get(name, 0) - before.get(name, 0) == 9, (tc, before, after)
    assert ops.device_errors(DEV) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [32, 64])
def test_a_far_key_among_hundreds(dtype, dim):
    """With a window that holds the whole sequence, one key hundreds of positions back (on another page, in
    another key tile, in another slice of a decoded row's keys) decides the output; at every page's border."""
    page = 16
    for distance in (200, 208, 209, 223, 224, 500):
        for lengths, new_rows, row in (((531, 40), (1, 1), 0), ((531, 40), (300, 2), 299)):
            out, want = _attention_case(dtype, 2, 1, dim, dim, 4000, 0, page, lengths, new_rows, seed=23, plant=(0, row, distance))
            a, b = out[0][row], want[0][row]
            tol = 1e-4 if dtype == torch.float32 else 2e-2
            assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), (distance, new_rows)
            assert float(b[:dim].abs().max()) > 5.0 and float(a[:dim].abs().max()) > 5.0, (distance, new_rows)


def test_the_fast_kernels_are_the_ones_that_run():
    from research_2_b200.kernels import ops

    before = ops.kernel_uses()
    _attention_case(torch.bfloat16, 4, 2, 32, 32, 44, 7, 16, (150, 37), (150, 2), seed=1)
    _attention_case(torch.bfloat16, 4, 2, 32, 32, 44, 7, 16, (150, 37), (1, 1), seed=1)
    _attention_case(torch.bfloat16, 3, 1, 24, 40, 9, 12, 4, (30, 7), (30, 2), seed=1)
    after = ops.kernel_uses()
    grew = {k: after.get(k, 0) - before.get(k, 0) for k in after}
    assert grew.get("attention_prefill", 0) == 1 and grew.get("attention_decode_fused", 0) == 1 and grew.get("attention_simt", 0) == 1, grew


# ---------------------------------------------------------------------------------------------
# whole models through the step function and the cache manager


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
    """Replays the trace in a pool of the trace's own peak demand plus one page (or `max_tokens`), filled
    with a loud value first. Returns ({step: logits}, how many pages had two owners or more)."""
    from research_2_b200.engine.replay import Replay

    live, round_to = traces.max_live(tb), 64
    if max_tokens is None:
        max_tokens, round_to = (traces.peak_pages(tb, page_size) + 1) * page_size, page_size
    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size, max_live=max(live, 1), round_to=round_to,
                    max_seq_len=max_seq_len)
    replay.step_fn.arena.fill_(64.0)
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
    if mode == "tiny_portions" and name == "c":
        pytest.skip("hundreds of steps; the other configurations cover portions of two tokens")
    folder, requests = folders[name], requests_for(name)
    tb = cut(requests, mode)
    outputs, reused, _ = run_trace(folder, tb, dtype, CASES[name]["page_size"])
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")
    if mode == "mixed":
        assert reused >= 4, f"only {reused} pages passed from one request to another"


def test_float32_logits_do_not_depend_on_the_cutting_at_all(folders):
    for name in ("a", "b", "d"):
        folder, requests = folders[name], requests_for(name)
        results = {}
        for mode in ("whole", "decode", "portions", "mixed"):
            tb = cut(requests, mode)
            results[mode] = compare(folder, requests, tb, run_trace(folder, tb, "float32", CASES[name]["page_size"])[0], "float32", f"{name}/{mode}")
        for mode in ("decode", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                for pos, logits in rows.items():
                    assert np.array_equal(logits, results[mode][rid][pos]), f"{name}: {mode} differs from whole at {rid}[{pos}]"


def test_a_window_group_gives_pages_back_and_keeps_the_first(folders):
    """While a long request decodes, its window group holds the pages of the kept first tokens and of the
    window only; the pool is far smaller than the sequence."""
    name = "a"
    folder, page = folders[name], CASES[name]["page_size"]
    ids = random_tokens(21, 400, CASES[name]["config"]["vocab"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=390)
    for dtype in ("float32", "bfloat16"):
        outputs, _, replay = run_trace(folder, tb, dtype, page, max_tokens=8 * page, max_seq_len=512)   # 400 tokens through 8 pages a group
        compare(folder, {"x": ids}, tb, outputs, dtype, f"long decoding in a small pool {dtype}")
        kinds = sorted((g.window, g.keep_first) for g in replay.cache.groups)
        assert kinds == [(17, 0), (24, 3)], kinds


def test_first_tokens(folders):
    for name in ("a", "b"):
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
    """Prompts of unequal length through `generate` (scheduler, portions under a small token budget, CUDA
    graphs): float32 tokens equal the plain implementation's; bfloat16 tokens are (nearly) the best by
    the plain logits of the sequence so far."""
    import research_2_b200

    name = "a"
    folder, vocab = folders[name], CASES[name]["config"]["vocab"]
    prompts = [random_tokens(40 + i, n, vocab) for i, n in enumerate((5, 61, 18, 33))]
    w, cfg = plain.read_model(folder, torch.float64)
    want = [plain.generate(w, cfg, p, 12) for p in prompts]
    got = research_2_b200.generate(folder, prompts, max_new_tokens=12, dtype="float32", device=DEV, block_size=8,
                                   max_batch_tokens=32, max_requests=3, max_seq_len=128)
    assert got == want, (got, want)
    got16 = research_2_b200.generate(folder, prompts, max_new_tokens=12, dtype="bfloat16", device=DEV, block_size=16,
                                     max_batch_tokens=48, max_requests=4, max_seq_len=128)
    for prompt, tokens in zip(prompts, got16):
        assert len(tokens) == 12
        logits = plain_logits(folder, (prompt + tokens)[:-1])
        slack = 2 * 2e-2 * float(np.abs(logits).max())
        for i, tok in enumerate(tokens):
            row = logits[len(prompt) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - slack, (i, tok)


def test_generation_in_a_pool_that_forces_preemption(folders):
    import research_2_b200

    name = "d"
    folder, vocab = folders[name], CASES[name]["config"]["vocab"]
    prompts = [random_tokens(60 + i, n, vocab) for i, n in enumerate((30, 44, 25))]
    w, cfg = plain.read_model(folder, torch.float64)
    want = [plain.generate(w, cfg, p, 10) for p in prompts]
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
    w, cfg = plain.read_model(folder, torch.float64)
    assert tokens == plain.generate(w, cfg, [5, 17, 3], 4)
