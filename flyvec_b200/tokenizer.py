"""Tokenizer objects the :class:`FlyVec` wrapper can sit on.

The reference's tokenizer (flyvec/tokenizer.py) is a text front-end built on
gensim and is not part of the accelerated path.  ``GensimTokenizer`` here only
loads a saved gensim dictionary when gensim is installed; ``VocabTokenizer``
offers the same four methods the hashing API needs (``tokenize``,
``token2id``, ``id2token``, ``n_vocab``) over a plain token list, with id 0
reserved for ``<UNK>`` as in the reference (flyvec/core.py:112-137).
"""
from __future__ import annotations

import re
from typing import Iterable, List


class VocabTokenizer:
    """Lower-cases, keeps ASCII word characters, looks tokens up in a list."""

    _split = re.compile(r"[a-z0-9_<>]+")

    def __init__(self, tokens: Iterable[str]):
        self.token_vocab: List[str] = list(tokens)
        if not self.token_vocab or self.token_vocab[0] != "<UNK>":
            self.token_vocab.insert(0, "<UNK>")
        self._ids = {t: i for i, t in enumerate(self.token_vocab)}
        self.vocab = self.token_vocab
        self.dictionary = self._ids

    @classmethod
    def from_file(cls, fname, phrases_file=None):
        with open(fname, "r", encoding="utf-8") as fp:
            return cls(line.rstrip("\n") for line in fp if line.strip())

    def tokenize(self, sentence: str) -> List[str]:
        return self._split.findall(sentence.lower())

    def token2id(self, token: str) -> int:
        return self._ids.get(token, 0)

    def id2token(self, tok_id: int) -> str:
        return self.token_vocab[tok_id]

    def n_vocab(self) -> int:
        return len(self.token_vocab)

    def encode(self, sentence: str) -> List[int]:
        return [self.token2id(t) for t in self.tokenize(sentence)]


class GensimTokenizer:
    """Loads the reference's saved gensim dictionary (flyvec/tokenizer.py:99-117).
    Requires gensim; everything else in this package works without it."""

    def __init__(self, dictionary, phrases=None):
        self.dictionary = dictionary
        self.phrases = phrases

    @classmethod
    def from_file(cls, dict_fname, phrases_fname=None):
        try:
            from gensim.corpora import Dictionary
            from gensim.models.phrases import Phraser
        except ImportError as e:  # pragma: no cover - gensim is optional
            raise ImportError("GensimTokenizer needs gensim; use VocabTokenizer for plain token lists") from e
        d = Dictionary.load(str(dict_fname))
        p = Phraser.load(str(phrases_fname)) if phrases_fname is not None else None
        return cls(d, p)

    @property
    def token_vocab(self):
        return list(self.dictionary.values())

    @property
    def vocab(self):
        return list(self.dictionary.keys())

    def n_vocab(self):
        return len(self.dictionary)

    def tokenize(self, sentence: str):
        toks = VocabTokenizer._split.findall(sentence.lower())
        return list(self.phrases[toks]) if self.phrases is not None else toks

    def token2id(self, token: str) -> int:
        return self.dictionary.token2id.get(token, 0)

    def id2token(self, tok_id: int) -> str:
        return self.dictionary[tok_id]
