"""The allocation-free token-hashing entry point (collected last on purpose, so a
failure here cannot hide another test's result in a run that stops at the first
failure).

fv_hash_tokens_static stages ids and codes in a fixed device array inside the
library instead of allocating per call; it exists for callers that hash small
batches next to a running trainer, or without any device memory of their own to
give.  It must return exactly what fv_hash_tokens returns, call after call, even
though every call reuses the same array with the previous call's leftovers in it."""
import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Hasher

pytestmark = pytest.mark.gpu


def test_static_staging_matches_allocating_path_twice_in_a_row(built_lib):
    K, V = 400, 1200
    W = synth.make_weights(K, 2 * V, seed=9)
    h = Hasher(W, normalize=True)
    # first call: a large batch in the reference's byte layout; second call: a smaller, different
    # batch, bit-packed, which lands on top of the first call's leftovers
    ids_a = synth.make_hash_ids(5000, V, seed=1)
    ids_b = synth.make_hash_ids(777, V, seed=2)
    for ids, hl, packed in ((ids_a, 50, False), (ids_b, 7, True)):
        want = h.hash_tokens(ids, hash_length=hl, packed=packed)
        got = h.hash_tokens_static(ids, hash_length=hl, packed=packed)
        assert got.dtype == want.dtype and got.shape == want.shape
        np.testing.assert_array_equal(got, want)  # bit-exact, the tolerance of every hashing test here
    # and the first batch again: nothing of the second call may leak into it
    np.testing.assert_array_equal(h.hash_tokens_static(ids_a, hash_length=50), h.hash_tokens(ids_a, hash_length=50))
    h.close()


def test_static_staging_allocates_nothing_and_matches_the_oracle(built_lib):
    """What the entry point is for: the device's free memory is the same before and after its calls
    (its first call on the device included, which only looks up the array's address), and its codes
    are the oracle's, compared directly."""
    from oracle import flyvec_oracle as orc

    K, V = 128, 600
    W = synth.make_weights(K, 2 * V, seed=12)
    h = Hasher(W, normalize=True)
    ids = synth.make_hash_ids(3000, V, seed=5)
    h.hash_tokens(ids[:16], hash_length=20)  # the hashing kernel itself is loaded by now (CUDA loads kernels on first use)
    free_before = _lib.device_free_bytes(0)
    first = h.hash_tokens_static(ids, hash_length=20)
    second = h.hash_tokens_static(ids[::-1].copy(), hash_length=20, packed=True)
    assert _lib.device_free_bytes(0) == free_before, "fv_hash_tokens_static changed the amount of free device memory"
    Wn = orc.normalize_synapses(W)
    np.testing.assert_array_equal(first, orc.hash_tokens(Wn, V, ids, 20))
    np.testing.assert_array_equal(second, orc.pack_codes(orc.hash_tokens(Wn, V, ids[::-1], 20)))
    h.close()


def test_static_staging_rejects_oversized_batches(built_lib):
    K, V = 400, 300
    h = Hasher(synth.make_weights(K, 2 * V, seed=3))
    limit = (Hasher.STATIC_SCRATCH_BYTES - 256) // (4 + K)  # byte layout: 4 bytes of id + K bytes of code per token
    ids = np.ones(limit + 1, np.int32)
    with pytest.raises(_lib.FlyvecError, match="fixed area holds"):
        h.hash_tokens_static(ids, hash_length=10)
    assert h.hash_tokens_static(ids[:limit], hash_length=10).shape == (limit, K)
    # bit-packed codes are 8x smaller, so the same batch plus more fits
    assert h.hash_tokens_static(np.ones(4 * limit, np.int32), hash_length=10, packed=True).shape == (4 * limit, 50)
    assert h.hash_tokens_static(np.zeros(0, np.int32), hash_length=10).shape == (0, K)
    h.close()
