"""``FlyVec``: the reference's hashing API (flyvec/core.py:39-211) over the CUDA hasher.

Constructor arguments, yaml keys, method names, return shapes and dtypes follow
the reference; the arithmetic (normalisation, activations, thresholding) runs
on the GPU through :class:`flyvec_b200.engine.Hasher`.  Batch methods are
additions.
"""
from __future__ import annotations

from functools import cached_property
from pathlib import Path
from typing import Dict, Optional, Union

import numpy as np

from .engine import Hasher
from .tokenizer import GensimTokenizer, VocabTokenizer

__all__ = ["softmax", "normalize_synapses", "FlyVec"]


def softmax(x: np.ndarray, beta: float = 1.0):
    """Softmax of a 1-D vector at inverse temperature ``beta`` (flyvec/core.py:17-20)."""
    v = np.exp(beta * x)
    return v / np.sum(v)


def normalize_synapses(syn: np.ndarray, prec: float = 1.0e-32, p: int = 2, device: int = 0) -> np.ndarray:
    """Rows of ``syn`` divided by their p-norm plus ``prec`` (flyvec/core.py:22-36),
    computed on the GPU with numpy's summation order; only ``p == 2`` exists there."""
    if p != 2:
        raise ValueError("only the 2-norm is implemented")
    h = Hasher(syn, normalize=True, prec=prec, device=device)
    try:
        return h.weights()
    finally:
        h.close()


class FlyVec:
    """Tokenizer + stop words + synapses for hashing words (flyvec/core.py:39-48)."""

    def __init__(self, synapse_file: Union[Path, str], tokenizer_file: Union[Path, str],
                 stopword_file: Optional[Union[Path, str]] = None, phrases_file: Optional[Union[Path, str]] = None,
                 normalize_synapses: bool = True, device: int = 0):
        self.synapse_file = str(synapse_file)
        self.tokenizer_file = str(tokenizer_file)
        self.stopword_file = str(stopword_file) if stopword_file is not None else None
        self.phrases_file = str(phrases_file) if phrases_file is not None else None
        self.normalize_synapses = normalize_synapses
        self.device = device

    @classmethod
    def load(cls, force_redownload=False):
        """Default model from the local cache directory (flyvec/core.py:50-59).  The
        reference downloads it when absent; this package has no network code, so a
        missing cache is an error."""
        cfg = Path.home() / ".cache" / "flyvec" / "data" / "config.yaml"
        if not cfg.exists():
            raise FileNotFoundError(f"{cfg} not found: place the pretrained model there or use FlyVec.from_config")
        return cls.from_config(cfg)

    @classmethod
    def from_config(cls, fname: Union[Path, str]):
        """Instance from a yaml file with keys ``synapses``, ``tokenizer`` and optionally
        ``phrases``, ``stop_words``, ``normalize_synapses`` (flyvec/core.py:62-77)."""
        import yaml

        fpath = Path(fname)
        ref_dir = fpath.parent
        with open(fname, "r") as fp:
            conf = yaml.load(fp, Loader=yaml.FullLoader)
        synapse_file = ref_dir / conf["synapses"]
        tokenizer_file = ref_dir / conf["tokenizer"]
        phrases_file = ref_dir / conf["phrases"] if "phrases" in conf.keys() else None
        stopword_file = ref_dir / conf["stop_words"] if "stop_words" in conf.keys() else None
        normalize = conf.get("normalize_synapses", False)
        return cls(synapse_file, tokenizer_file, stopword_file=stopword_file, phrases_file=phrases_file,
                   normalize_synapses=normalize)

    # -- model state ---------------------------------------------------------
    @cached_property
    def hasher(self) -> Hasher:
        syn = np.load(self.synapse_file)
        return Hasher(syn, normalize=self.normalize_synapses, device=self.device)

    @cached_property
    def n_neurons(self):
        return self.hasher.K

    @cached_property
    def synapses(self):
        """The (normalised, if requested) weights as a host array."""
        return self.hasher.weights()

    @cached_property
    def tokenizer(self):
        if self.tokenizer_file.endswith(".txt"):
            return VocabTokenizer.from_file(self.tokenizer_file)
        return GensimTokenizer.from_file(self.tokenizer_file, self.phrases_file)

    @cached_property
    def dictionary(self):
        return self.tokenizer.dictionary

    @cached_property
    def vocab(self):
        return self.tokenizer.vocab

    @cached_property
    def token_vocab(self):
        return self.tokenizer.token_vocab

    @cached_property
    def n_vocab(self):
        return self.tokenizer.n_vocab()

    @cached_property
    def stop_word_ids(self):
        return set(np.load(self.stopword_file))

    @cached_property
    def stop_words(self):
        return set([self.tokenizer.id2token(t) for t in self.stop_word_ids])

    @cached_property
    def unknown_embedding_info(self):
        return {"token": "<UNK>", "id": 0, "embedding": np.zeros(self.n_neurons).astype(np.uint8)}

    # -- per-word API (flyvec/core.py:127-185) --------------------------------
    def tokenize(self, sentence: str):
        return self.tokenizer.tokenize(sentence)

    def is_unknown_token(self, token: str):
        if len(token) == 0:
            raise ValueError("Token cannot be the empty string")
        tok = self.tokenizer.tokenize(token)[0]
        tok_id = self.tokenizer.token2id(tok)
        return tok_id == 0

    def get_sparse_embedding(self, word: str, hash_length: int = 50):
        """Context-independent binary code of the first token of ``word``:
        ``{'token', 'id', 'embedding': int8[K]}``; unknown words give zeros."""
        if self.is_unknown_token(word):
            return self.unknown_embedding_info
        token = self.tokenizer.tokenize(word)[0]
        tok_id = self.tokenizer.token2id(token)
        if hash_length >= self.n_neurons:
            raise IndexError(f"hash_length {hash_length} is out of bounds for {self.n_neurons} neurons")
        code = self.hasher.hash_tokens([tok_id], hash_length=hash_length)[0]
        return {"token": token, "id": tok_id, "embedding": code}

    def get_dense_embedding(self, word: str):
        if self.is_unknown_token(word):
            return self.unknown_embedding_info
        token = self.tokenizer.tokenize(word)[0]
        tok_id = self.tokenizer.token2id(token)
        return {"token": token, "id": tok_id, "embedding": self.synapses[:, self.n_vocab + tok_id]}

    def simple_word_vectors(self, k: int = 50, exclude_stop_words=False, output_list=False) -> Dict[str, np.ndarray]:
        """Codes of the whole vocabulary at hash length ``k`` (flyvec/core.py:187-211),
        hashed in one batch."""
        toks = list(self.token_vocab)
        ids = np.array([self.tokenizer.token2id(t) for t in toks], dtype=np.int32)
        codes = self.hasher.hash_tokens(ids, hash_length=k)
        stop = self.stop_words if exclude_stop_words else ()
        out = {}
        for t, c in zip(toks, codes):
            if exclude_stop_words and t in stop:
                continue
            out[t] = list(c) if output_list else c
        return out

    def save_simple_word_vectors(self, fname, k: int = 51, exclude_stop_words: bool = False) -> int:
        """Write the context-independent codes of the whole vocabulary as JSON, ``{token: [0/1, ...]}`` --
        the shape of the reference's precomputed ``simple-flyvec-embeddings.json`` (README, "Simple word
        embeddings", hash length 51).  Returns the number of tokens written."""
        import json

        vecs = self.simple_word_vectors(k=k, exclude_stop_words=exclude_stop_words)
        with open(fname, "w") as fp:
            json.dump({t: [int(x) for x in v] for t, v in vecs.items()}, fp)
        return len(vecs)

    # -- batch additions ------------------------------------------------------
    def get_sparse_embeddings(self, ids, hash_length: int = 50, packed: bool = False) -> np.ndarray:
        """Codes for an array of token ids: int8 ``[n][K]`` or bit-packed uint8 ``[n][ceil(K/8)]``."""
        return self.hasher.hash_tokens(ids, hash_length=hash_length, packed=packed)

    def hash_windows(self, idx, inv_freq=None, hash_length: int = 50, packed: bool = False) -> np.ndarray:
        """Context-dependent codes of windows of input ids (centre id offset by the
        vocabulary size), weighted by ``inv_freq`` when given."""
        return self.hasher.hash_windows(idx, inv_freq=inv_freq, hash_length=hash_length, packed=packed)
