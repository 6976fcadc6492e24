"""Small Bosenex configurations for the tests, model folders with random weights, and the plain implementation's
logits with an error budget.

The configurations differ from one another in every size and constant, and between them cover the values that one
model may happen to make equal or trivial: layers in every order (matrix memories only: a model without any
per-token cache; side-by-side layers only), one head and several, as many key/value heads as query heads and a
single one, value heads smaller and larger than key heads, head sizes that are no multiple of 16, a rotation of a
part of a head and none, capped and uncapped scores and gates, a window of a few tokens, one longer than any
sequence and none, convolutions of one to four taps, one group and several for B/C and for the norm, layers
without a feed-forward, experts of which one, some or all are used, with and without the expert that every token
uses, clamps that bite and clamps that never do, a state matrix whose columns are spread over several CTAs.
"""

from __future__ import annotations

import functools
from pathlib import Path

import numpy as np
import torch

from tests.plain import bosenex_plain


def memory(heads, dim, vdim, cap=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap is not None:
        m["gate_cap"] = cap
    return m


def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def space(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp=None):
    kind = "parallel" if "left" in mixer else "mlstm"
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6, embedding_scale=None, logit_scale=None):
    cfg = {"architecture": "Bosenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embedding_scale is not None:
        cfg["embedding"] = {"scale": embedding_scale}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


CASES = {
    # every kind of layer and of feed-forward, a layer without one
    "a": {"config": model(211, 64, [
        layer({"left": attention(4, 2, 16, 16, 0.3, window=24, rot=(16, 10000.0), softcap=20.0), "right": space(2, 16, 8, 1, 4, 1)}, dense(96)),
        layer(memory(2, 16, 16, cap=10.0), moe(4, 2, 32, 1.0, shared=(48, 2.0))),
        layer(memory(4, 8, 24, cap=3.0)),
        layer({"left": attention(2, 2, 32, 8, 0.2, window=7, rot=(8, 500.0)), "right": space(4, 8, 16, 4, 2, 2)}, moe(3, 3, 16, 0.3)),
    ], eps=1e-6, embedding_scale=4.0, logit_scale=0.5), "seed": 3, "std": 0.08, "page_size": 16},
    # side-by-side layers only; sizes that only the general kernels take; one expert per token
    "b": {"config": model(97, 40, [
        layer({"left": attention(3, 1, 24, 40, 0.25, window=9, rot=(12, 77.0)), "right": space(4, 10, 12, 2, 3, 4)}, moe(5, 1, 24, 50.0)),
        layer({"left": attention(1, 1, 20, 12, 0.5, window=1, softcap=5.0), "right": space(1, 40, 5, 1, 1, 1)}, dense(56)),
    ], eps=2e-5), "seed": 5, "std": 0.1, "page_size": 8},
    # matrix memories only (no per-token cache at all); a state of 64 x 128 whose columns two CTAs share; uncapped gates
    "c": {"config": model(300, 128, [
        layer(memory(1, 64, 128), dense(160)),
        layer(memory(8, 16, 8, cap=15.0), moe(6, 2, 24, 1.5, shared=(16, 0.5))),
    ], eps=1e-5, embedding_scale=8.0, logit_scale=2.0), "seed": 8, "std": 0.05, "page_size": 32},
    # key and value heads of 64, no window in one layer and one beyond every sequence in the other, full rotation, pages of 4
    "d": {"config": model(128, 96, [
        layer({"left": attention(2, 1, 64, 64, 0.125, rot=(64, 10000.0), softcap=30.0), "right": space(3, 32, 24, 3, 4, 3)}),
        layer(memory(3, 24, 40, cap=8.0), dense(72)),
        layer({"left": attention(4, 4, 64, 64, 0.11, window=100000), "right": space(2, 48, 64, 1, 2, 1)}, moe(2, 1, 40, 2.0, shared=(8, 1.0))),
    ], eps=1e-5, embedding_scale=1.0, logit_scale=1.0), "seed": 13, "std": 0.07, "page_size": 4},
}


def _divisors(n: int) -> list[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def random_case(seed: int) -> dict:
    """A configuration drawn from a seed: one to five layers of either kind in any order, sizes that are and are not
    multiples of 16, every optional mechanism there or not."""
    import random

    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            mixer = memory(rng.randint(1, 6), rng.choice([4, 8, 12, 16, 24, 32, 48, 64, 96]), rng.choice([4, 8, 16, 20, 32, 48, 64, 96, 128]),
                           cap=rng.choice([None, 5.0, 15.0, 30.0]))
        else:
            heads = rng.randint(1, 8)
            dim = rng.choice([8, 16, 24, 32, 48, 64, 80, 96, 128])
            rot = None
            if rng.random() < 0.8:
                rot = (rng.choice(list(range(2, dim + 1, 2))) if rng.random() < 0.4 else dim, rng.choice([100.0, 10000.0, 500000.0]))
            left = attention(heads, rng.choice(_divisors(heads)), dim, rng.choice([dim, dim, 8, 16, 32, 40, 64]), rng.choice([dim ** -0.5, 0.1, 0.3]),
                             window=rng.choice([None, 1, 3, 16, 17, 64, 100, 136, 1000]), rot=rot, softcap=rng.choice([None, 10.0, 30.0, 50.0]))
            s_heads, s_vdim = rng.randint(1, 6), rng.choice([4, 8, 16, 24, 32, 48, 64])
            right = space(s_heads, s_vdim, rng.choice([4, 8, 16, 32, 64, 128]), rng.choice(_divisors(s_heads)), rng.randint(1, 4),
                          rng.choice(_divisors(s_heads * s_vdim)[:6]))
            mixer = {"left": left, "right": right}
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.45:
            mlp = dense(rng.choice([16, 40, 64, 96, 200]))
        else:
            experts = rng.randint(2, 12)
            mlp = moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 16, 24, 32, 64]), rng.choice([0.5, 1.0, 7.0]),
                      shared=(rng.choice([8, 16, 48]), rng.choice([0.5, 1.5])) if rng.random() < 0.6 else None)
        layers.append(layer(mixer, mlp))
    config = model(rng.choice([50, 97, 256, 1000]), rng.choice([24, 40, 64, 72, 100, 128, 192, 320]), layers, eps=rng.choice([1e-6, 1e-5]),
                   embedding_scale=rng.choice([None, 1.0, 4.0, 16.0]), logit_scale=rng.choice([None, 0.25, 1.0, 2.0]))
    return {"config": config, "seed": seed, "std": 0.06, "page_size": rng.choice([4, 8, 16, 32]), "length": rng.choice([40, 150, 300])}


def make_model_dir(folder: Path, case: dict, store_dtype: str = "bfloat16") -> Path:
    from research_2_b200 import models  # noqa: F401  (registers the architectures)
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.weights import write_model_folder

    arch = architecture_of(case["config"])
    return write_model_folder(folder, arch, arch.parse_config(case["config"]), case["seed"], store_dtype, std=case["std"])


def random_tokens(seed: int, n: int, vocab: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, ids: tuple) -> np.ndarray:
    cfg, w = bosenex_plain.read_model(folder)
    return bosenex_plain.forward(cfg, w, list(ids)).numpy()


def plain_logits(folder, ids) -> np.ndarray:
    return _plain_cached(str(folder), tuple(int(i) for i in ids))


@functools.lru_cache(maxsize=64)
def _movement_cached(folder: str, ids: tuple) -> np.ndarray:
    """Per position, how far the plain logits move when every normalised row is disturbed by relative noise of 2^-9
    (about bfloat16's rounding, which the engine applies in more places), the most over eight draws. Large where the design itself is discontinuous or
    ill-conditioned: a matrix memory whose first q . k is nearly zero and is then normalised. A position at which a router's
    choice hangs on less than a hundredth of |h| |w| is excused altogether (infinity)."""
    cfg, w = bosenex_plain.read_model(folder)
    truth = _plain_cached(folder, ids)
    worst = np.zeros(len(ids))
    bosenex_plain.MARGINS = []
    try:
        bosenex_plain.forward(cfg, w, list(ids))
        for margin in bosenex_plain.MARGINS:
            worst[margin.numpy() < 0.01] = np.inf   # a close call of a router: either choice is right at 16-bit precision
    finally:
        bosenex_plain.MARGINS = None
    for seed in range(8):
        gen = torch.Generator().manual_seed(1000 + seed)
        bosenex_plain.DISTURB = lambda x: x * (1 + 2.0 ** -9 * torch.randn(x.shape, generator=gen, dtype=torch.float64))
        try:
            moved = bosenex_plain.forward(cfg, w, list(ids)).numpy()
        finally:
            bosenex_plain.DISTURB = None
        worst = np.maximum(worst, np.abs(moved - truth).max(axis=1))
    return worst


FLOORS = {"float32": 3e-5, "bfloat16": 3e-2}


def assert_close_to_plain(got: np.ndarray, folder, ids, dtype_name: str, positions=None, what: str = "") -> None:
    """|logit - truth| <= floor * max |truth| with truth in float64; floors 3e-5 (float32) and 3e-2 (bfloat16). In
    bfloat16 a position may also be off by three times what disturbances of the size of its rounding do to the plain logits
    there: positions at which the design is discontinuous are so excused, and only those."""
    truth = plain_logits(folder, ids)
    allowed = np.full(len(truth), FLOORS[dtype_name] * float(np.abs(truth).max()))
    if dtype_name == "bfloat16":
        allowed = np.maximum(allowed, 3.0 * _movement_cached(str(folder), tuple(int(i) for i in ids)))
    if positions is not None:
        truth, allowed = truth[list(positions)], allowed[list(positions)]
    assert got.shape == truth.shape, (got.shape, truth.shape, what)
    err = np.abs(got.astype(np.float64) - truth).max(axis=1)
    if not bool((err <= allowed).all()):
        first_bad = int(np.argmax(~(err <= allowed)))
        pos = list(positions)[first_bad] if positions is not None else first_bad
        raise AssertionError(f"{what}: |logit - truth| = {float(err[first_bad]):.3e} > allowed {float(allowed[first_bad]):.3e} at "
                             f"position {pos}, the first of {int((~(err <= allowed)).sum())} positions over their limit")
