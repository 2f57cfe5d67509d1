"""Text transforms and vocabularies for ``Dataset.map``: tokenizers (whitespace, unicode character / script, regex,
basic, wordpiece, BERT, SentencePiece, user function), ``Vocab`` / ``Lookup``, pretrained-vector tables
(``Vectors``, ``GloVe``, ``FastText``, ``CharNGram``) with ``ToVectors``, and the sequence helpers (``Ngram``,
``SlidingWindow``, ``Truncate``, ``TruncateSequencePair``, ``AddToken``, ``ToNumber``, ``CaseFold``,
``NormalizeUTF8``, ``RegexReplace``, ``FilterWikipediaXML``).  Inputs and outputs are numpy arrays of str.

Parity: python/mindspore/dataset/text/transforms.py, utils.py."""
from __future__ import annotations

import enum
import re
import unicodedata

import numpy as np


class JiebaMode(enum.IntEnum):
    MIX, MP, HMM = 0, 1, 2


class NormalizeForm(enum.IntEnum):
    NONE, NFC, NFKC, NFD, NFKD = 0, 1, 2, 3, 4


class SentencePieceModel(enum.IntEnum):
    UNIGRAM, BPE, CHAR, WORD = 0, 1, 2, 3


class SPieceTokenizerOutType(enum.IntEnum):
    STRING, INT = 0, 1


class SPieceTokenizerLoadType(enum.IntEnum):
    FILE, MODEL = 0, 1


def to_str(array, encoding="utf8"):
    a = np.asarray(array)
    if a.dtype.kind in ("U", "O"):
        return a.astype(str)
    return np.char.decode(a, encoding)


def to_bytes(array, encoding="utf8"):
    return np.char.encode(np.asarray(array).astype(str), encoding)


def _s(x):
    a = np.asarray(x)
    if a.ndim != 0:
        raise RuntimeError("the input must be a scalar string, but got shape %s" % (a.shape,))
    v = a.item()
    return v.decode() if isinstance(v, bytes) else str(v)


def _arr(tokens):
    return np.array(list(tokens), dtype=object).astype(str) if len(tokens) else np.array([], dtype=str)


def _with_offsets(text, tokens, with_offsets):
    out = _arr(tokens)
    if not with_offsets:
        return out
    starts, limits, pos = [], [], 0
    data = text.encode()
    for t in tokens:
        b = t.encode()
        i = data.find(b, pos)
        i = pos if i < 0 else i
        starts.append(i)
        limits.append(i + len(b))
        pos = i + len(b)
    return out, np.array(starts, dtype=np.uint32), np.array(limits, dtype=np.uint32)


class TextTensorOperation:
    """Base of the text transforms."""

    def __call__(self, *inputs):
        return self._run(*inputs)


# ---------------------------------------------------------------------------------------------------- vocabulary
class Vocab:
    """Token <-> id table; build it with ``from_list`` / ``from_dict`` / ``from_file`` / ``from_dataset``."""

    def __init__(self):
        self._tok2id, self._id2tok = {}, []

    @classmethod
    def _build(cls, words, special_tokens, special_first):
        v = cls()
        special = list(special_tokens or [])
        seq = (special + list(words)) if special_first else (list(words) + special)
        for w in seq:
            if w in v._tok2id:
                raise ValueError("word_list contains duplicate word: %s." % w)
            v._tok2id[w] = len(v._id2tok)
            v._id2tok.append(w)
        return v

    @classmethod
    def from_list(cls, word_list, special_tokens=None, special_first=True):
        if special_tokens and set(special_tokens) & set(word_list):
            raise ValueError("special_tokens and word_list contain duplicate word.")
        return cls._build(word_list, special_tokens, special_first)

    @classmethod
    def from_dict(cls, word_dict):
        v = cls()
        ids = sorted(word_dict.values())
        if ids != list(range(len(ids))) and len(set(ids)) != len(ids):
            raise ValueError("word ids must be unique")
        for w, i in sorted(word_dict.items(), key=lambda kv: kv[1]):
            v._tok2id[w] = i
        v._id2tok = [None] * (max(ids) + 1 if ids else 0)
        for w, i in word_dict.items():
            v._id2tok[i] = w
        return v

    @classmethod
    def from_file(cls, file_path, delimiter="", vocab_size=None, special_tokens=None, special_first=True):
        words = []
        with open(file_path, encoding="utf-8") as f:
            for ln in f:
                ln = ln.rstrip("\n")
                if not ln:
                    continue
                words.append(ln.split(delimiter)[0] if delimiter else ln)
                if vocab_size and len(words) >= vocab_size:
                    break
        return cls._build(words, special_tokens, special_first)

    @classmethod
    def from_dataset(cls, dataset, columns=None, freq_range=None, top_k=None, special_tokens=None, special_first=True):
        """Words of the given columns ordered by falling frequency (ties alphabetically), filtered by
        ``freq_range`` = (min, max) and cut to ``top_k``."""
        from collections import Counter
        cols = [columns] if isinstance(columns, str) else list(columns or dataset.get_col_names())
        counts = Counter()
        for row in dataset.create_dict_iterator(output_numpy=True, num_epochs=1):
            for c in cols:
                counts.update(str(t) for t in np.asarray(row[c]).reshape(-1))
        lo, hi = (freq_range or (None, None))
        words = [w for w, n in sorted(counts.items(), key=lambda kv: (-kv[1], kv[0]))
                 if (lo is None or n >= lo) and (hi is None or n <= hi)]
        return cls._build(words[:top_k] if top_k else words, special_tokens, special_first)

    def vocab(self):
        return dict(self._tok2id)

    def tokens_to_ids(self, tokens):
        if isinstance(tokens, str):
            return self._tok2id.get(tokens, -1)
        return [self._tok2id.get(str(t), -1) for t in tokens]

    def ids_to_tokens(self, ids):
        def one(i):
            if i < 0:
                raise ValueError("The single id should be no less than 0.")
            return self._id2tok[i] if i < len(self._id2tok) and self._id2tok[i] is not None else ""
        return one(ids) if isinstance(ids, (int, np.integer)) else [one(int(i)) for i in ids]

    def __len__(self):
        return len(self._tok2id)


class Lookup(TextTensorOperation):
    def __init__(self, vocab, unknown_token=None, data_type=np.int32):
        self.vocab, self.dtype = vocab, np.dtype(data_type) if not hasattr(data_type, "is_floating_point") else np.int32
        self.unk = None
        if unknown_token is not None:
            self.unk = vocab.tokens_to_ids(unknown_token)
            if self.unk < 0:
                raise RuntimeError("Lookup: unknown_token %r is not in the vocabulary" % (unknown_token,))

    def _run(self, x):
        a = np.asarray(x)
        flat = []
        for t in a.reshape(-1):
            i = self.vocab.tokens_to_ids(str(t))
            if i < 0:
                if self.unk is None:
                    raise RuntimeError("Lookup: token %r is not in the vocabulary and no unknown_token was given"
                                       % (str(t),))
                i = self.unk
            flat.append(i)
        return np.array(flat, dtype=self.dtype).reshape(a.shape)


class Vectors:
    """A table of pretrained word vectors read from a text file: ``token v1 v2 ...`` per line (a first line of two
    integers - count and dimension - is skipped)."""

    def __init__(self):
        self.table, self.dim = {}, 0

    @classmethod
    def from_file(cls, file_path, max_vectors=None):
        v = cls()
        with open(file_path, encoding="utf-8") as f:
            for k, ln in enumerate(f):
                parts = ln.rstrip().split(" ")
                if k == 0 and len(parts) == 2 and all(p.isdigit() for p in parts):
                    continue
                if len(parts) < 2:
                    continue
                v.table[parts[0]] = np.array([float(p) for p in parts[1:]], dtype=np.float32)
                if max_vectors and len(v.table) >= max_vectors:
                    break
        v.dim = len(next(iter(v.table.values()))) if v.table else 0
        return v


class GloVe(Vectors):
    """``glove.*.txt`` tables."""


class FastText(Vectors):
    """``*.vec`` tables."""


class CharNGram(Vectors):
    """Character n-gram tables (entries look like ``3gram-abc``): a word's vector is the mean of the vectors of its
    n-grams (with ``#BEGIN#`` / ``#END#`` markers) that are in the table."""

    def lookup_word(self, word):
        chars = ["#BEGIN#"] + list(word) + ["#END#"]
        found = []
        for n in (2, 3, 4):
            for i in range(len(chars) - n + 1):
                key = "%dgram-%s" % (n, "".join(chars[i:i + n]))
                if key in self.table:
                    found.append(self.table[key])
        return np.mean(found, 0).astype(np.float32) if found else None


class ToVectors(TextTensorOperation):
    def __init__(self, vectors, unk_init=None, lower_case_backup=False):
        self.vectors, self.lower = vectors, lower_case_backup
        self.unk = np.asarray(unk_init, dtype=np.float32) if unk_init is not None else np.zeros(vectors.dim,
                                                                                               np.float32)
        if self.unk.shape != (vectors.dim,):
            raise ValueError("ToVectors: unk_init must have %d entries" % vectors.dim)

    def _one(self, t):
        v = self.vectors.table.get(t)
        if v is None and self.lower:
            v = self.vectors.table.get(t.lower())
        if v is None and isinstance(self.vectors, CharNGram):
            v = self.vectors.lookup_word(t)
        return self.unk if v is None else v

    def _run(self, x):
        a = np.asarray(x)
        if a.ndim == 0:
            return self._one(str(a.item()))
        return np.stack([self._one(str(t)) for t in a.reshape(-1)])


# ---------------------------------------------------------------------------------------------------- tokenizers
class WhitespaceTokenizer(TextTensorOperation):
    def __init__(self, with_offsets=False):
        self.with_offsets = with_offsets

    def _run(self, x):
        text = _s(x)
        return _with_offsets(text, text.split(), self.with_offsets)


class UnicodeCharTokenizer(TextTensorOperation):
    def __init__(self, with_offsets=False):
        self.with_offsets = with_offsets

    def _run(self, x):
        text = _s(x)
        return _with_offsets(text, list(text), self.with_offsets)


def _script(ch):
    if ch.isspace():
        return "space"
    cat = unicodedata.category(ch)
    if cat.startswith("P") or cat.startswith("S"):
        return "punct"
    if cat.startswith("N"):
        return "digit"
    name = unicodedata.name(ch, "")
    return name.split(" ")[0] if name else "other"


class UnicodeScriptTokenizer(TextTensorOperation):
    """Splits where the Unicode script (approximated by the first word of the character name) changes."""

    def __init__(self, keep_whitespace=False, with_offsets=False):
        self.keep, self.with_offsets = keep_whitespace, with_offsets

    def _run(self, x):
        text = _s(x)
        tokens, cur, last = [], "", None
        for ch in text:
            sc = _script(ch)
            if sc != last and cur:
                tokens.append((cur, last))
                cur = ""
            cur, last = cur + ch, sc
        if cur:
            tokens.append((cur, last))
        out = [t for t, sc in tokens if self.keep or sc != "space"]
        return _with_offsets(text, out, self.with_offsets)


class RegexTokenizer(TextTensorOperation):
    """Splits at ``delim_pattern``; delimiters matching ``keep_delim_pattern`` are kept as tokens."""

    def __init__(self, delim_pattern, keep_delim_pattern="", with_offsets=False):
        self.delim, self.keep = re.compile(delim_pattern), re.compile(keep_delim_pattern) if keep_delim_pattern else None
        self.with_offsets = with_offsets

    def _run(self, x):
        text = _s(x)
        tokens, pos = [], 0
        for m in self.delim.finditer(text):
            if m.start() > pos:
                tokens.append(text[pos:m.start()])
            if self.keep is not None and self.keep.fullmatch(m.group(0)) and m.group(0):
                tokens.append(m.group(0))
            pos = m.end()
        if pos < len(text):
            tokens.append(text[pos:])
        return _with_offsets(text, tokens, self.with_offsets)


class RegexReplace(TextTensorOperation):
    def __init__(self, pattern, replace, replace_all=True):
        self.pattern, self.replace, self.count = re.compile(pattern), replace, 0 if replace_all else 1

    def _run(self, x):
        a = np.asarray(x)
        f = np.vectorize(lambda t: self.pattern.sub(self.replace, str(t), count=self.count), otypes=[object])
        return f(a).astype(str) if a.ndim else np.array(self.pattern.sub(self.replace, _s(a), count=self.count))


class CaseFold(TextTensorOperation):
    def _run(self, x):
        a = np.asarray(x)
        return np.vectorize(lambda t: str(t).casefold(), otypes=[object])(a).astype(str)


class NormalizeUTF8(TextTensorOperation):
    def __init__(self, normalize_form=NormalizeForm.NFKC):
        self.form = {0: None, 1: "NFC", 2: "NFKC", 3: "NFD", 4: "NFKD"}[int(normalize_form)]

    def _run(self, x):
        if self.form is None:
            return np.asarray(x).astype(str)
        return np.vectorize(lambda t: unicodedata.normalize(self.form, str(t)), otypes=[object])(np.asarray(x)).astype(
            str)


class FilterWikipediaXML(TextTensorOperation):
    """Keeps letters a-z and spaces of the text content of Wikipedia XML (markup, tags, references and digits
    removed, upper case folded), like the classic ``wikifil`` clean-up of enwik9."""

    def _run(self, x):
        t = _s(x)
        t = re.sub(r"<[^>]*>", " ", t)
        t = re.sub(r"&[a-z]+;", " ", t)
        t = re.sub(r"\[\[[^\]|]*\|", "[[", t)
        t = re.sub(r"\{\{[^}]*\}\}|\[http[^\]]*\]", " ", t)
        for d, w in zip("0123456789", ("zero", "one", "two", "three", "four", "five", "six", "seven", "eight",
                                       "nine")):
            t = t.replace(d, " %s " % w)
        t = re.sub(r"[^a-z]+", " ", t.lower())
        return np.array(t.strip())


class BasicTokenizer(TextTensorOperation):
    """BERT's first stage: optional lower-casing + accent stripping, whitespace split, every punctuation mark and
    CJK character becomes a token of its own; ``preserve_unused_token`` keeps ``[UNK]``-like tokens whole."""

    _SPECIAL = re.compile(r"\[(?:CLS|SEP|UNK|MASK|PAD|unused\d+)\]")

    def __init__(self, lower_case=False, keep_whitespace=False, normalization_form=NormalizeForm.NONE,
                 preserve_unused_token=True, with_offsets=False):
        self.lower, self.keep_ws, self.norm = lower_case, keep_whitespace, NormalizeUTF8(normalization_form)
        self.preserve, self.with_offsets = preserve_unused_token, with_offsets

    @staticmethod
    def _is_cjk(ch):
        c = ord(ch)
        return 0x4E00 <= c <= 0x9FFF or 0x3400 <= c <= 0x4DBF or 0xF900 <= c <= 0xFAFF or 0x20000 <= c <= 0x2FA1F

    def _split(self, word):
        if self.preserve and self._SPECIAL.fullmatch(word):
            return [word]
        if self.lower:
            word = "".join(c for c in unicodedata.normalize("NFD", word.lower()) if unicodedata.category(c) != "Mn")
        out, cur = [], ""
        for ch in word:
            cat = unicodedata.category(ch)
            if cat.startswith("P") or cat.startswith("S") or self._is_cjk(ch):
                if cur:
                    out.append(cur)
                out.append(ch)
                cur = ""
            else:
                cur += ch
        if cur:
            out.append(cur)
        return out

    def tokenize(self, text):
        text = str(self.norm._run(np.array(text)))
        tokens = []
        for piece in re.split(r"(\s+)", text):
            if not piece:
                continue
            if piece.isspace():
                if self.keep_ws:
                    tokens.append(piece)
                continue
            if self.preserve:
                pos = 0
                for m in self._SPECIAL.finditer(piece):
                    tokens += self._split(piece[pos:m.start()]) if m.start() > pos else []
                    tokens.append(m.group(0))
                    pos = m.end()
                tokens += self._split(piece[pos:]) if pos < len(piece) else []
            else:
                tokens += self._split(piece)
        return tokens

    def _run(self, x):
        text = _s(x)
        return _with_offsets(text.lower() if self.lower else text, self.tokenize(text), self.with_offsets)


class WordpieceTokenizer(TextTensorOperation):
    """Greedy longest-match-first split of every input token into vocabulary pieces (continuations prefixed)."""

    def __init__(self, vocab, suffix_indicator="##", max_bytes_per_token=100, unknown_token="[UNK]",
                 with_offsets=False):
        self.vocab, self.suffix, self.max_bytes, self.unk = vocab, suffix_indicator, max_bytes_per_token, unknown_token
        self.with_offsets = with_offsets

    def pieces(self, token):
        if len(token.encode()) > self.max_bytes:
            return [self.unk or token]
        out, start = [], 0
        while start < len(token):
            end, cur = len(token), None
            while start < end:
                sub = (self.suffix if start > 0 else "") + token[start:end]
                if self.vocab.tokens_to_ids(sub) >= 0:
                    cur = sub
                    break
                end -= 1
            if cur is None:
                return [self.unk or token]
            out.append(cur)
            start = end
        return out

    def _run(self, x):
        toks = [str(t) for t in np.asarray(x).reshape(-1)]
        out = [p for t in toks for p in self.pieces(t)]
        if not self.with_offsets:
            return _arr(out)
        starts, limits = [], []
        for t in toks:
            pos = 0
            for p in self.pieces(t):
                n = len(t.encode()) if p == self.unk else len(p[len(self.suffix):].encode() if p.startswith(
                    self.suffix) and pos else p.encode())
                starts.append(pos)
                limits.append(pos + n)
                pos += n
        return _arr(out), np.array(starts, np.uint32), np.array(limits, np.uint32)


class BertTokenizer(TextTensorOperation):
    """``BasicTokenizer`` followed by ``WordpieceTokenizer``."""

    def __init__(self, vocab, suffix_indicator="##", max_bytes_per_token=100, unknown_token="[UNK]", lower_case=False,
                 keep_whitespace=False, normalization_form=NormalizeForm.NONE, preserve_unused_token=True,
                 with_offsets=False):
        self.basic = BasicTokenizer(lower_case, keep_whitespace, normalization_form, preserve_unused_token)
        self.wordpiece = WordpieceTokenizer(vocab, suffix_indicator, max_bytes_per_token, unknown_token)
        self.with_offsets = with_offsets

    def _run(self, x):
        text = _s(x)
        words = self.basic.tokenize(text)
        pieces = [p for w in words for p in self.wordpiece.pieces(w)]
        if not self.with_offsets:
            return _arr(pieces)
        _, ws, _ = _with_offsets(text.lower() if self.basic.lower else text, words, True)
        starts, limits = [], []
        for w, base in zip(words, ws.tolist()):
            pos = base
            for p in self.wordpiece.pieces(w):
                body = p[len(self.wordpiece.suffix):] if p.startswith(self.wordpiece.suffix) and pos > base else p
                n = len(w.encode()) if p == self.wordpiece.unk else len(body.encode())
                starts.append(pos)
                limits.append(pos + n)
                pos += n
        return _arr(pieces), np.array(starts, np.uint32), np.array(limits, np.uint32)


class PythonTokenizer(TextTensorOperation):
    def __init__(self, tokenizer):
        if not callable(tokenizer):
            raise TypeError("`tokenizer` is not a callable Python function")
        self.fn = tokenizer

    def _run(self, x):
        try:
            return _arr([str(t) for t in self.fn(_s(x))])
        except Exception as e:  # noqa: BLE001
            raise RuntimeError("Error occurred in Pyfunc [%s]." % getattr(self.fn, "__name__", "tokenizer")) from e


class JiebaTokenizer(TextTensorOperation):
    """Chinese word segmentation with the ``jieba`` package's dictionaries (``hmm_path`` / ``mp_path`` are the
    dictionary files of cppjieba in the reference; here the package must be importable)."""

    def __init__(self, hmm_path, mp_path, mode=JiebaMode.MIX, with_offsets=False):
        try:
            import jieba
        except ImportError as e:
            raise RuntimeError("JiebaTokenizer needs the 'jieba' package, which is not installed") from e
        self.jieba, self.mode, self.with_offsets = jieba, JiebaMode(mode), with_offsets
        self.words = {}

    def add_word(self, word, freq=None):
        self.jieba.add_word(word, freq)

    def add_dict(self, user_dict):
        items = user_dict.items() if isinstance(user_dict, dict) else []
        for w, f in items:
            self.add_word(w, f)

    def _run(self, x):
        text = _s(x)
        toks = list(self.jieba.cut(text, HMM=self.mode != JiebaMode.MP))
        return _with_offsets(text, toks, self.with_offsets)


class SentencePieceVocab:
    """A SentencePiece model: trained from text files (``from_file`` / ``from_dataset``) or loaded
    (``load_model``); ``save_model`` writes it."""

    def __init__(self, model_bytes=None):
        self.model_bytes = model_bytes

    @classmethod
    def from_file(cls, file_path, vocab_size, character_coverage, model_type, params):
        import io

        import sentencepiece as spm
        kind = {0: "unigram", 1: "bpe", 2: "char", 3: "word"}[int(model_type)]
        buf = io.BytesIO()
        spm.SentencePieceTrainer.train(input=",".join(file_path), model_writer=buf, vocab_size=vocab_size,
                                       character_coverage=character_coverage, model_type=kind,
                                       minloglevel=2, **{k: v for k, v in (params or {}).items()})
        return cls(buf.getvalue())

    @classmethod
    def from_dataset(cls, dataset, col_names, vocab_size, character_coverage, model_type, params):
        import os
        import tempfile
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "corpus.txt")
            with open(path, "w", encoding="utf-8") as f:
                for row in dataset.create_dict_iterator(output_numpy=True, num_epochs=1):
                    for c in col_names:
                        for t in np.asarray(row[c]).reshape(-1):
                            f.write(str(t) + "\n")
            return cls.from_file([path], vocab_size, character_coverage, model_type, params)

    @classmethod
    def load_model(cls, path):
        with open(path, "rb") as f:
            return cls(f.read())

    @classmethod
    def save_model(cls, vocab, path, filename):
        import os
        with open(os.path.join(path, filename), "wb") as f:
            f.write(vocab.model_bytes)


class SentencePieceTokenizer(TextTensorOperation):
    def __init__(self, mode, out_type):
        import sentencepiece as spm
        if isinstance(mode, SentencePieceVocab):
            self.sp = spm.SentencePieceProcessor(model_proto=mode.model_bytes)
        elif isinstance(mode, str):
            self.sp = spm.SentencePieceProcessor(model_file=mode)
        else:
            raise TypeError("SentencePieceTokenizer: 'mode' must be a SentencePieceVocab or a model file path")
        self.out_int = int(out_type) == int(SPieceTokenizerOutType.INT)

    def _run(self, x):
        text = _s(x)
        if self.out_int:
            return np.array(self.sp.encode(text, out_type=int), dtype=np.int32)
        return _arr(self.sp.encode(text, out_type=str))


# ---------------------------------------------------------------------------------------------------- sequence helpers
class Ngram(TextTensorOperation):
    """All n-grams (for every n of ``n``) of a 1-D token array, joined by ``separator``; ``left_pad`` / ``right_pad``
    = (token, width) pad the sequence first."""

    def __init__(self, n, left_pad=("", 0), right_pad=("", 0), separator=" "):
        self.ns = [n] if isinstance(n, int) else list(n)
        if any(k <= 0 for k in self.ns):
            raise ValueError("Ngram: every n must be positive")
        self.left, self.right, self.sep = left_pad, right_pad, separator

    def _run(self, x):
        toks = [str(t) for t in np.asarray(x).reshape(-1)]
        out = []
        for n in self.ns:
            seq = [self.left[0]] * min(self.left[1], n - 1) + toks + [self.right[0]] * min(self.right[1], n - 1)
            out += [self.sep.join(seq[i:i + n]) for i in range(len(seq) - n + 1)]
        return _arr(out)


class SlidingWindow(TextTensorOperation):
    def __init__(self, width, axis=0):
        if width <= 0:
            raise ValueError("SlidingWindow: width must be positive")
        self.width, self.axis = width, axis

    def _run(self, x):
        a = np.asarray(x)
        if a.ndim != 1 or self.axis not in (0, -1):
            raise RuntimeError("SlidingWindow supports 1-D input with axis 0")
        n = a.shape[0] - self.width + 1
        if n <= 0:
            return a[:0].reshape(0, self.width)
        return np.stack([a[i:i + self.width] for i in range(n)])


class Truncate(TextTensorOperation):
    def __init__(self, max_seq_len):
        if max_seq_len < 0:
            raise ValueError("Truncate: max_seq_len must be non-negative")
        self.n = max_seq_len

    def _run(self, x):
        a = np.asarray(x)
        return a[..., :self.n]


class TruncateSequencePair(TextTensorOperation):
    """Trims two sequences so that their total length is at most ``max_length``, removing from the longer one."""

    def __init__(self, max_length):
        self.n = max_length

    def _run(self, a, b):
        a, b = np.asarray(a), np.asarray(b)
        la, lb = len(a), len(b)
        while la + lb > self.n:
            if la > lb:
                la -= 1
            else:
                lb -= 1
        return a[:la], b[:lb]


class AddToken(TextTensorOperation):
    def __init__(self, token, begin=True):
        self.token, self.begin = token, begin

    def _run(self, x):
        a = np.asarray(x).astype(str)
        tok = np.full(a.shape[:-1] + (1,), self.token)
        return np.concatenate([tok, a] if self.begin else [a, tok], -1).astype(str)


class ToNumber(TextTensorOperation):
    def __init__(self, data_type):
        self.dtype = np.dtype(data_type) if not hasattr(data_type, "is_floating_point") else np.dtype(
            str(data_type).replace("torch.", ""))
        if self.dtype.kind not in "iuf":
            raise TypeError("ToNumber: data_type must be a numeric type, but got %s" % (data_type,))

    def _run(self, x):
        a = np.asarray(x)
        try:
            vals = np.vectorize(lambda t: float(str(t)) if self.dtype.kind == "f" else int(str(t)), otypes=[object])(a)
        except ValueError as e:
            raise RuntimeError("ToNumber: %s" % e) from e
        if self.dtype.kind in "iu":
            info = np.iinfo(self.dtype)
            if any(int(v) < info.min or int(v) > info.max for v in np.asarray(vals).reshape(-1)):
                raise RuntimeError("ToNumber: a value is out of the range of %s" % self.dtype)
        return np.asarray(vals).astype(self.dtype)


__all__ = [n for n, v in list(globals().items()) if not n.startswith("_") and (
    (isinstance(v, type) and v.__module__ == __name__) or n in ("to_str", "to_bytes"))]
