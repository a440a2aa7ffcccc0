"""Tokenizers.

* ``CLIPTokenizer``: lower-cased, whitespace-cleaned text, regex pre-tokenisation, BPE over byte-mapped characters with
  the end-of-word marker ``</w>``, ``<|startoftext|>`` / ``<|endoftext|>`` framing, padding to 77 (vocab.json +
  merges.txt) (serenitymojo/tokenizer/clip_tokenizer.mojo).
* ``ByteLevelBPE``: GPT-2 style byte-level BPE with the Qwen pre-tokenisation pattern and special tokens kept atomic
  (vocab.json + merges.txt, or the ``model`` section of a tokenizer.json) (serenitymojo/tokenizer/tokenizer.mojo).
* ``T5Tokenizer``: SentencePiece unigram model through the ``sentencepiece`` library, appending ``</s>``
  (serenitymojo/tokenizer/t5_tokenizer.mojo)."""
from __future__ import annotations

import json
import re
from functools import lru_cache
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


@lru_cache()
def bytes_to_unicode() -> Dict[int, str]:
    """Reversible byte -> printable unicode character map (printable bytes map to themselves)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


def _pairs(word: Sequence[str]):
    return {(a, b) for a, b in zip(word[:-1], word[1:])}


class _BPE:
    def __init__(self, vocab: Dict[str, int], merges: Iterable[Tuple[str, str]]):
        self.encoder = vocab
        self.decoder = {v: k for k, v in vocab.items()}
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.cache: Dict[str, List[str]] = {}

    def bpe(self, symbols: Tuple[str, ...]) -> List[str]:
        key = "\x00".join(symbols)
        if key in self.cache:
            return self.cache[key]
        word = list(symbols)
        while len(word) > 1:
            best = min(_pairs(word), key=lambda p: self.ranks.get(p, 1 << 60))
            if best not in self.ranks:
                break
            a, b = best
            out, i = [], 0
            while i < len(word):
                if i < len(word) - 1 and word[i] == a and word[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = out
        self.cache[key] = word
        return word


def _read_merges(path: str) -> List[Tuple[str, str]]:
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line or line.startswith("#version"):
                continue
            a, b = line.split(" ")
            out.append((a, b))
    return out


class CLIPTokenizer:
    PAT = re.compile(r"<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[a-zA-ZÀ-ɏ]+|[0-9]|[^\sa-zA-Z0-9À-ɏ]+",
                     re.IGNORECASE)

    def __init__(self, vocab: Dict[str, int], merges: Iterable[Tuple[str, str]], max_length: int = 77, pad_with_eos: bool = True):
        self.bpe = _BPE(vocab, merges)
        self.b2u = bytes_to_unicode()
        self.sot, self.eot = vocab["<|startoftext|>"], vocab["<|endoftext|>"]
        self.max_length = max_length
        self.pad_id = self.eot if pad_with_eos else 0

    @classmethod
    def from_files(cls, vocab_json: str, merges_txt: str, **kw):
        return cls(json.load(open(vocab_json, encoding="utf-8")), _read_merges(merges_txt), **kw)

    def tokenize(self, text: str) -> List[int]:
        text = re.sub(r"\s+", " ", text).strip().lower()
        ids = []
        for tok in self.PAT.findall(text):
            chars = [self.b2u[b] for b in tok.encode("utf-8")]
            chars[-1] += "</w>"
            ids += [self.bpe.encoder[p] for p in self.bpe.bpe(tuple(chars))]
        return ids

    def __call__(self, text: str) -> Tuple[List[int], List[int]]:
        ids = [self.sot] + self.tokenize(text)[: self.max_length - 2] + [self.eot]
        mask = [1] * len(ids) + [0] * (self.max_length - len(ids))
        return ids + [self.pad_id] * (self.max_length - len(ids)), mask

    def decode(self, ids: Sequence[int]) -> str:
        u2b = {v: k for k, v in self.b2u.items()}
        text = "".join(self.bpe.decoder[i] for i in ids if i not in (self.sot, self.eot))
        words = [bytearray(u2b[c] for c in w).decode("utf-8", "replace") for w in text.split("</w>")]
        return " ".join(words).strip()


class ByteLevelBPE:
    PAT = re.compile(r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\w]?[^\W\d_]+|\d| ?[^\s\w]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+", re.UNICODE)

    def __init__(self, vocab: Dict[str, int], merges: Iterable[Tuple[str, str]], special_tokens: Optional[Dict[str, int]] = None):
        self.bpe = _BPE(vocab, merges)
        self.b2u = bytes_to_unicode()
        self.special = dict(special_tokens or {})
        self.special_re = re.compile("(" + "|".join(re.escape(s) for s in sorted(self.special, key=len, reverse=True)) + ")") if self.special else None
        self.id_to_special = {v: k for k, v in self.special.items()}

    @classmethod
    def from_files(cls, vocab_json: str, merges_txt: str, special_tokens=None):
        return cls(json.load(open(vocab_json, encoding="utf-8")), _read_merges(merges_txt), special_tokens)

    @classmethod
    def from_tokenizer_json(cls, path: str):
        d = json.load(open(path, encoding="utf-8"))
        merges = [tuple(m.split(" ")) if isinstance(m, str) else tuple(m) for m in d["model"]["merges"]]
        special = {t["content"]: t["id"] for t in d.get("added_tokens", [])}
        return cls(d["model"]["vocab"], merges, special)

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        parts = self.special_re.split(text) if self.special_re else [text]
        for part in parts:
            if not part:
                continue
            if part in self.special:
                ids.append(self.special[part])
                continue
            for tok in self.PAT.findall(part):
                sym = tuple(self.b2u[b] for b in tok.encode("utf-8"))
                ids += [self.bpe.encoder[p] for p in self.bpe.bpe(sym)]
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        u2b = {v: k for k, v in self.b2u.items()}
        out = bytearray()
        for i in ids:
            if i in self.id_to_special:
                out += self.id_to_special[i].encode("utf-8")
            else:
                out += bytes(u2b[c] for c in self.bpe.decoder[i])
        return out.decode("utf-8", "replace")

    def chat_template(self, prompt: str, system: str = "") -> str:
        """The instruct framing the Qwen-family encoders are fed with."""
        sys_part = f"<|im_start|>system\n{system}<|im_end|>\n" if system else ""
        return f"{sys_part}<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"


class T5Tokenizer:
    def __init__(self, model_file: str, max_length: int = 512):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=model_file)
        self.max_length = max_length
        self.eos = self.sp.eos_id() if self.sp.eos_id() >= 0 else 1
        self.pad = self.sp.pad_id() if self.sp.pad_id() >= 0 else 0

    def __call__(self, text: str, pad: bool = True) -> Tuple[List[int], List[int]]:
        ids = self.sp.encode(text)[: self.max_length - 1] + [self.eos]
        mask = [1] * len(ids)
        if pad:
            mask += [0] * (self.max_length - len(ids))
            ids += [self.pad] * (self.max_length - len(ids))
        return ids, mask
