"""Bit-exact parity of the CUDA hasher with the oracle's restatement of
flyvec/core.py:22-36, 139-185 and with the golden vectors produced by the
reference's own code.  All calls go through the C ABI."""
from pathlib import Path

import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Hasher
from oracle import flyvec_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("K,V", [(400, 600), (64, 100), (100, 333), (130, 50), (1000, 64)])
def test_normalisation_is_bit_exact(built_lib, K, V):
    W = synth.make_weights(K, 2 * V, seed=K + V)
    h = Hasher(W, normalize=True)
    np.testing.assert_array_equal(h.weights(), orc.normalize_synapses(W))
    h.close()
    h = Hasher(W, normalize=False)
    np.testing.assert_array_equal(h.weights(), W)
    h.close()


@pytest.mark.parametrize("K,V,normalize", [(400, 2000, True), (400, 2000, False), (100, 300, True), (70, 90, False)])
@pytest.mark.parametrize("hash_length", [1, 4, 16, 50])
def test_token_codes_bit_exact(built_lib, K, V, normalize, hash_length):
    W = synth.make_weights(K, 2 * V, seed=3)
    ids = synth.make_hash_ids(3000, V, seed=17)
    syn = orc.normalize_synapses(W) if normalize else W
    ref = orc.hash_tokens(syn, V, ids, hash_length)
    h = Hasher(W, normalize=normalize)
    got = h.hash_tokens(ids, hash_length=hash_length)
    assert got.dtype == np.int8 and got.shape == (ids.size, K)
    np.testing.assert_array_equal(got, ref)
    packed = h.hash_tokens(ids, hash_length=hash_length, packed=True)
    np.testing.assert_array_equal(packed, orc.pack_codes(ref))
    assert not got[ids == 0].any()
    h.close()


def test_token_codes_with_ties(built_lib):
    """Quantised weights make equal activations common: the strict '>' against the
    midpoint then yields fewer than hash_length ones (flyvec/core.py:155-158)."""
    rng = np.random.default_rng(5)
    K, V = 128, 200
    W = rng.integers(-3, 4, size=(K, 2 * V)).astype(np.float32)
    ids = np.arange(V, dtype=np.int32)
    h = Hasher(W, normalize=False)
    for hl in (1, 7, 50, 127):
        ref = orc.hash_tokens(W, V, ids, hl)
        np.testing.assert_array_equal(h.hash_tokens(ids, hash_length=hl), ref)
        assert (ref.sum(axis=1) <= hl).all() and (ref.sum(axis=1) < hl).any()
    h.close()


@pytest.mark.parametrize("weighted", [True, False])
@pytest.mark.parametrize("hash_length", [4, 50, 200])
def test_window_codes_bit_exact(built_lib, weighted, hash_length):
    K, V, W = 400, 1500, 11
    enc, off = synth.make_corpus(30000, V, seed=23)
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=False)
    Wm = orc.normalize_synapses(synth.make_weights(K, 2 * V, seed=4))
    idx = orc.build_idx(enc, starts, np.arange(0, 4000), W, V)
    idx[5, 3] = -1  # a padded position
    ref = orc.hash_windows(Wm, V, idx, f if weighted else None, hash_length)
    h = Hasher(Wm, normalize=False)
    got = h.hash_windows(idx, inv_freq=f if weighted else None, hash_length=hash_length)
    np.testing.assert_array_equal(got, ref)
    packed = h.hash_windows(idx, inv_freq=f if weighted else None, hash_length=hash_length, packed=True)
    np.testing.assert_array_equal(packed, orc.pack_codes(ref))
    h.close()


def test_window_codes_certified_and_exact_pass_agree(built_lib):
    """Float window sums are only trusted when the two order statistics around the threshold are far
    enough apart; ties and close calls must fall back to the reference's double arithmetic.  Weights
    quantised to a few levels make exact ties and near-ties common."""
    K, V, W = 200, 600, 9
    rng = np.random.default_rng(5)
    Wm = (rng.integers(-3, 4, (K, 2 * V)) * np.float32(0.25)).astype(np.float32)
    Wm[:, ::7] += np.float32(1e-6) * rng.standard_normal((K, Wm[:, ::7].shape[1])).astype(np.float32)
    enc, off = synth.make_corpus(20000, V, seed=29)
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=False)
    idx = orc.build_idx(enc, starts, np.arange(0, 3000), W, V)
    h = Hasher(Wm, normalize=False)
    for inv in (None, f):
        for hl in (1, 16, 50):
            ref = orc.hash_windows(Wm, V, idx, inv, hl)
            np.testing.assert_array_equal(h.hash_windows(idx, inv_freq=inv, hash_length=hl), ref)
            np.testing.assert_array_equal(h.hash_windows(idx, inv_freq=inv, hash_length=hl, exact=True), ref)
    h.close()


def test_golden_vectors_from_reference(built_lib):
    """Codes the reference's unmodified FlyVec.get_sparse_embedding produced for a
    seeded matrix (tests/golden/make_hash_golden.py)."""
    g = np.load(GOLDEN / "hash_golden.npz")
    W = synth.make_weights(int(g["K"]), 2 * int(g["V"]), seed=int(g["seed"]))
    for normalize, key in ((True, "codes_norm"), (False, "codes_raw")):
        h = Hasher(W, normalize=normalize)
        for hl, codes in zip(g["hash_lengths"], g[key]):
            got = h.hash_tokens(g["ids"], hash_length=int(hl))
            np.testing.assert_array_equal(got, codes)
        h.close()


def test_hash_errors(built_lib):
    W = synth.make_weights(16, 40, seed=1)
    h = Hasher(W)
    with pytest.raises(_lib.FlyvecError, match="hash_length"):
        h.hash_tokens([1, 2], hash_length=16)  # the reference raises IndexError here
    with pytest.raises(_lib.FlyvecError, match="out of range"):
        h.hash_tokens([1, 25], hash_length=4)
    assert h.hash_tokens(np.zeros(0, np.int32), hash_length=4).shape == (0, 16)
    h.close()
    with pytest.raises(ValueError):
        Hasher(np.zeros((4, 7), np.float32))


def test_flyvec_api_matches_reference_shapes(built_lib, tmp_path):
    """The drop-in class: dict results, dtypes, unknown-word behaviour
    (nbs/00_core.ipynb test cells: default hash length 50, case-insensitive,
    first token of a phrase, empty string raises)."""
    from flyvec_b200 import FlyVec

    K, V = 64, 50
    W = synth.make_weights(K, 2 * V, seed=2)
    words = ["<UNK>"] + [f"w{i}" for i in range(1, V)]
    np.save(tmp_path / "syn.npy", W)
    (tmp_path / "vocab.txt").write_text("\n".join(words))
    (tmp_path / "config.yaml").write_text("synapses: syn.npy\ntokenizer: vocab.txt\nnormalize_synapses: true\n")
    m = FlyVec.from_config(tmp_path / "config.yaml")
    e = m.get_sparse_embedding("w7")
    syn = orc.normalize_synapses(W)
    assert e["token"] == "w7" and e["id"] == 7 and e["embedding"].dtype == np.int8
    np.testing.assert_array_equal(e["embedding"], orc.threshold_code(syn[:, V + 7], 50))
    assert e["embedding"].sum() == 50
    np.testing.assert_array_equal(m.get_sparse_embedding("W7")["embedding"], e["embedding"])
    np.testing.assert_array_equal(m.get_sparse_embedding("w7 w9")["embedding"], e["embedding"])
    assert m.get_sparse_embedding("w7", hash_length=4)["embedding"].sum() == 4
    unk = m.get_sparse_embedding("notaword")
    assert unk["token"] == "<UNK>" and unk["embedding"].dtype == np.uint8 and not unk["embedding"].any()
    with pytest.raises(ValueError, match="empty string"):
        m.get_sparse_embedding("")
    np.testing.assert_array_equal(m.get_dense_embedding("w7")["embedding"], syn[:, V + 7])
    vecs = m.simple_word_vectors(k=10)
    assert len(vecs) == V and vecs["w3"].sum() == 10
    import json

    assert m.save_simple_word_vectors(tmp_path / "simple.json", k=12) == V
    dumped = json.loads((tmp_path / "simple.json").read_text())
    assert sorted(dumped) == sorted(words) and sum(dumped["w3"]) == 12 and len(dumped["w3"]) == K
    assert dumped["<UNK>"] == [0] * K
