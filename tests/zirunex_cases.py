"""Small Zirunex configurations for the tests, model folders with random weights, and the plain
implementation's logits with an error budget.

The configurations differ from one another in every size and constant, and between them cover the values
that one model may happen to make equal or trivial: as many key/value heads as query heads and a single
one, one query head, a window longer than any test sequence and a window of one, no kept first tokens and
more kept tokens than a window holds, value heads smaller and larger than key heads, a head size that is
no multiple of 16, layers without a feed-forward, layers that run with another layer's tensors (the lender
before and after other layers), clamps that bite and clamps that never do.
"""

from __future__ import annotations

import functools
from pathlib import Path

import numpy as np
import torch

from tests.plain import zirunex_plain


def _mixer(heads, kv_heads, dim, vdim, window, keep_first, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "keep_first": keep_first}}


def _layer(mixer, ff=None, limit=None, weights_of=None):
    entry = {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


_A0 = _mixer(4, 2, 16, 16, 24, 3, 0.31)
_A1 = _mixer(2, 2, 32, 32, 17, 0, 0.2)
_B0 = _mixer(3, 1, 24, 40, 9, 12, 0.25)       # a head size that is no multiple of 16; values wider than keys
_B1 = _mixer(1, 1, 32, 16, 1, 2, 0.5)         # one head; a window of one; values narrower than keys
_C0 = _mixer(8, 1, 64, 64, 70, 5, 0.125)      # eight query heads on one key/value head
_C1 = _mixer(2, 1, 64, 64, 100000, 7, 0.11)   # a window longer than any sequence: every key is seen
_D0 = _mixer(4, 4, 32, 32, 33, 64, 0.2)       # kept first tokens reach over a page's and a tile's border

CASES = {
    # head sizes of 16 and 32, grouped and ungrouped heads, a layer without a feed-forward, a borrower at the end
    "a": {"config": {"architecture": "Zirunex", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.5},
                     "layers": [_layer(_A0, 96, 1.5), _layer(_A1), _layer(_A0, 96, 1.5, weights_of=0)]},
          "seed": 3, "std": 0.08, "page_size": 16},
    # shapes that only the general kernel takes; a borrower between its lender and another layer
    "b": {"config": {"architecture": "Zirunex", "vocab": 97, "width": 40, "norm": {"eps": 2e-5}, "embedding": {"scale": 0.7},
                     "layers": [_layer(_B0, 56, 0.4), _layer(_B0, 56, 0.4, weights_of=0), _layer(_B1, 24, 50.0)]},
          "seed": 5, "std": 0.15, "page_size": 8},
    # head size 64 and prompts of several 64-row tiles
    "c": {"config": {"architecture": "Zirunex", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
                     "layers": [_layer(_C0, 160, 2.5), _layer(_C1, 64, 1.0), _layer(_C1, 64, 1.0, weights_of=1),
                                _layer(_C0, 160, 2.5, weights_of=0)]},
          "seed": 8, "std": 0.05, "page_size": 32},
    "d": {"config": {"architecture": "Zirunex", "vocab": 128, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
                     "layers": [_layer(_D0, 128, 3.0), _layer(_D0)]},
          "seed": 13, "std": 0.07, "page_size": 4},
}


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
def _plain_cached(folder: str, ids: tuple, dtype_name: str) -> np.ndarray:
    dtype = {"float32": torch.float32, "float64": torch.float64}[dtype_name]
    w, cfg = zirunex_plain.read_model(folder, dtype)
    return zirunex_plain.forward(w, cfg, torch.tensor(ids)).numpy()


def plain_logits(folder, ids, dtype_name: str = "float64") -> np.ndarray:
    return _plain_cached(str(folder), tuple(int(i) for i in ids), dtype_name)


FLOORS = {"float32": 2e-5, "bfloat16": 2e-2}


def assert_close_to_plain(got: np.ndarray, folder, ids, dtype_name: str, positions=None, what: str = "") -> None:
    """|logit - truth| <= max(2 * the plain implementation's own float32 error, floor * max |truth|), truth
    in float64; floors 2e-5 (float32) and 2e-2 (bfloat16)."""
    truth = plain_logits(folder, ids, "float64")
    err_ref = float(np.abs(plain_logits(folder, ids, "float32") - truth).max())
    allowed = max(2.0 * err_ref, FLOORS[dtype_name] * float(np.abs(truth).max()))
    if positions is not None:
        truth = truth[list(positions)]
    assert got.shape == truth.shape, (got.shape, truth.shape, what)
    err = np.abs(got.astype(np.float64) - truth)
    if not float(err.max()) <= allowed:
        first_bad = int(np.argmax(err.max(axis=1) > allowed))
        pos = list(positions)[first_bad] if positions is not None else first_bad
        raise AssertionError(f"{what}: max |logit - truth| = {float(err.max()):.3e} > allowed {allowed:.3e}; "
                             f"the first position over it is {pos}")
