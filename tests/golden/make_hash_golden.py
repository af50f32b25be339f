"""Generates tests/golden/hash_golden.npz by running the reference's own hashing code.

Run from the repository root in a container that has the reference checkout:

    python tests/golden/make_hash_golden.py /path/to/reference
    python tests/golden/make_hash_golden.py /path/to/reference --time   # only times the reference's hashing

The reference's ``flyvec/core.py`` is imported unchanged.  Its third-party
imports that are not needed for hashing (cached_property, fastcore, gensim,
boto3, progressbar) are replaced by stub modules; the synapse matrix and a
minimal tokenizer are injected into a ``FlyVec`` instance, and the real
``FlyVec.get_sparse_embedding`` and ``normalize_synapses`` produce the codes.
The matrix is regenerated in the tests from the stored seed
(``flyvec_b200.synth.make_weights``), so only ids and codes are stored.
"""
import sys
import types
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))


def import_reference(ref_root: str):
    class cached_property:  # stores the value in the instance dict, like the real one
        def __init__(self, fn):
            self.fn, self.name = fn, fn.__name__

        def __get__(self, obj, cls):
            if obj is None:
                return self
            val = obj.__dict__[self.name] = self.fn(obj)
            return val

    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    stub("cached_property", cached_property=cached_property)
    stub("fastcore")
    stub("fastcore.test")
    stub("fastcore.script")
    stub("boto3")
    stub("botocore")
    stub("progressbar")
    stub("gensim")
    stub("gensim.corpora", Dictionary=object)
    stub("gensim.models")
    stub("gensim.models.phrases", Phrases=object, Phraser=object)
    stub("gensim.parsing")
    stub("gensim.parsing.preprocessing", strip_punctuation=None, strip_multiple_whitespaces=None)
    sys.path.insert(0, ref_root)
    try:
        from flyvec.core import FlyVec, normalize_synapses
    except Exception:
        # tokenizer.py / downloader.py may import names the stubs lack: stub those modules whole
        for k in [k for k in sys.modules if k.startswith("flyvec")]:
            del sys.modules[k]
        stub("flyvec.tokenizer", GensimTokenizer=object)
        stub("flyvec.downloader", prepare_flyvec_data=None, get_config_dir=None, get_model_dir=None)
        from flyvec.core import FlyVec, normalize_synapses
    return FlyVec, normalize_synapses


class FakeTokenizer:
    def __init__(self, V):
        self.V = V

    def tokenize(self, s):
        return s.split()

    def token2id(self, t):
        return int(t[1:]) if t.startswith("t") and t[1:].isdigit() and int(t[1:]) < self.V else 0

    def n_vocab(self):
        return self.V


def time_reference(FlyVec, normalize_synapses, n_tokens: int = 20000):
    """Throughput of the reference's own per-token hashing on config-0 shapes (K=400, V=20000, hash_length 50),
    one core, wherever this script runs (the reference checkout does not travel to a GPU box)."""
    import time
    from flyvec_b200 import synth

    K, V = 400, 20000
    model = FlyVec("unused.npy", "unused.dict", normalize_synapses=True)
    model.__dict__["synapses"] = normalize_synapses(synth.make_weights(K, 2 * V, seed=1))
    model.__dict__["tokenizer"] = FakeTokenizer(V)
    words = [f"t{t}" for t in synth.make_hash_ids(n_tokens, V, seed=100)]
    t0 = time.perf_counter()
    for w in words:
        model.get_sparse_embedding(w, hash_length=50)
    dt = time.perf_counter() - t0
    print(f"reference FlyVec.get_sparse_embedding: {n_tokens} tokens in {dt:.2f} s = {n_tokens / dt:.0f} tokens/s (1 core)")


def main():
    from oracle.build_oracle import reference_root

    ref = reference_root(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else None)
    if ref is None:
        raise SystemExit("no reference checkout: pass its path, or set FLYVEC_REFERENCE")
    ref_root = str(ref)
    FlyVec, normalize_synapses = import_reference(ref_root)
    from flyvec_b200 import synth

    if "--time" in sys.argv:
        return time_reference(FlyVec, normalize_synapses)

    K, V, seed = 128, 300, 4242
    hash_lengths = np.array([1, 8, 50], dtype=np.int32)
    W = synth.make_weights(K, 2 * V, seed=seed)
    ids = synth.make_hash_ids(400, V, seed=77)
    ids[:5] = [0, 1, V - 1, 2, 0]
    out = {}
    for key, norm in (("codes_norm", True), ("codes_raw", False)):
        model = FlyVec("unused.npy", "unused.dict", normalize_synapses=norm)
        model.__dict__["synapses"] = normalize_synapses(W) if norm else W
        model.__dict__["tokenizer"] = FakeTokenizer(V)
        codes = np.zeros((len(hash_lengths), ids.size, K), dtype=np.int8)
        for a, hl in enumerate(hash_lengths):
            for n, t in enumerate(ids):
                emb = model.get_sparse_embedding(f"t{t}", hash_length=int(hl))["embedding"]
                codes[a, n] = emb
        out[key] = codes
    np.savez_compressed(Path(__file__).resolve().parent / "hash_golden.npz", K=K, V=V, seed=seed, ids=ids,
                        hash_lengths=hash_lengths, **out)
    print("wrote hash_golden.npz", {k: v.shape for k, v in out.items()},
          "ones per code (norm, hl=50):", out["codes_norm"][2].sum(axis=1)[:8])


if __name__ == "__main__":
    main()
