"""The C-ABI shared library: it builds for sm_100a without a GPU, loads, and
exports every function include/flyvec_b200.h declares.  Host-side entry points
(window enumeration, inverse frequency, shard arithmetic) are exercised; nothing
here touches a device."""
import re
from pathlib import Path

import numpy as np
import pytest

from flyvec_b200 import _lib, engine
from oracle import flyvec_oracle as orc

HEADER = Path(__file__).resolve().parent.parent / "include" / "flyvec_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fv_[a-z0-9_]+)\s*\(", text)))


def test_header_and_library_agree(built_lib):
    names = declared_functions()
    assert len(names) >= 35
    for n in names:
        assert hasattr(built_lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib._PROTOTYPES), "ctypes prototypes out of step with the header"
    assert built_lib.fv_version() == 1


def test_config_struct_size():
    # 14 four-byte fields
    import ctypes

    assert ctypes.sizeof(_lib.FvConfig) == 56
    assert ctypes.sizeof(_lib.FvRunStats) == 72


@pytest.mark.parametrize("W", [1, 5, 11])
def test_host_window_enumeration_matches_oracle(built_lib, W):
    rng = np.random.default_rng(W + 100)
    lens = np.concatenate([rng.integers(0, 60, 3000), [213, 214, 215, 1000, W, W - 1]])
    rng.shuffle(lens)
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)
    np.testing.assert_array_equal(engine.enumerate_windows(off, W), orc.enumerate_windows(off, W))
    assert len(engine.enumerate_windows(np.array([0], np.uint64), W)) == 0


def test_host_inverse_frequency_matches_oracle(built_lib):
    rng = np.random.default_rng(3)
    enc = rng.integers(-1, 500, 200000).astype(np.int32)
    np.testing.assert_array_equal(engine.inverse_frequency(enc, 600), orc.inverse_word_frequency(enc, 600))
    with pytest.raises(_lib.FlyvecError, match="token id"):
        engine.inverse_frequency(np.array([700], np.int32), 600)


def test_shard_ranges_tile_the_order(built_lib):
    ns, batch, world = 10_345, 100, 4
    seen = np.zeros(ns, np.int32)
    steps = (ns + batch * world - 1) // (batch * world)
    for step in range(steps):
        for r in range(world):
            first, count = engine.shard_range(ns, batch, world, r, step)
            assert count <= batch
            seen[first:first + count] += 1
    assert (seen == 1).all()
    assert engine.shard_range(ns, batch, world, 0, steps)[1] == 0
    with pytest.raises(_lib.FlyvecError):
        engine.shard_range(ns, batch, 2, 2, 0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(FileNotFoundError, match="no CPU fallback"):
        _lib.lib()
