"""CPU tests of the byte-level BPE tokenizer (Gpt2Tokenizer, tokenizer.rs:34-62).  The r50k_base
vocabulary is data that is not available offline, so the algorithm is pinned on a synthetic merge table
against a third statement of it in pure Python (tiktoken's published byte_pair_merge), on the round-trip
property decode(encode(text)) == text, and on GPT-2's split pattern."""
import base64

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

import b200nn
from b200nn import Gpt2Tokenizer, TokenizerError
from b200nn.tokenizer import GPT2_SPLIT_PATTERN


def _table():
    """256 single bytes (in a shuffled order, as r50k_base's are) and merges learnt greedily from a small
    corpus: every merge joins two existing tokens, ranks in order of creation."""
    rng = np.random.default_rng(3)
    order = rng.permutation(256)
    ranks = {bytes([int(b)]): i for i, b in enumerate(order)}
    corpus = (b" the quick brown fox jumps over the lazy dog and the other dogs don't mind; they're asleep. "
              b"1234 5678 2024 12 hello hello world worlds wording  \n\n\tthe end   of the thing's things!!! ??? "
              + "naïve café über straße 中文 日本".encode())
    words = [list(bytes([b]) for b in w) for w in corpus.split(b" ") if w]
    words = [[b" "] + w for w in words]
    for _ in range(200):
        counts = {}
        for w in words:
            for a, b in zip(w, w[1:]):
                counts[(a, b)] = counts.get((a, b), 0) + 1
        if not counts:
            break
        (a, b), c = max(counts.items(), key=lambda kv: (kv[1], kv[0]))
        if c < 2:
            break
        ranks[a + b] = len(ranks)
        new = []
        for w in words:
            i, o = 0, []
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    o.append(a + b)
                    i += 2
                else:
                    o.append(w[i])
                    i += 1
            new.append(o)
        words = new
    return ranks


def _py_merge(ranks, piece: bytes):
    """tiktoken's byte_pair_merge, as published: merge the adjacent pair of lowest rank until none is left."""
    if piece in ranks:
        return [ranks[piece]]
    parts = [bytes([b]) for b in piece]
    while len(parts) > 1:
        best, bi = None, -1
        for i in range(len(parts) - 1):
            r = ranks.get(parts[i] + parts[i + 1])
            if r is not None and (best is None or r < best):
                best, bi = r, i
        if best is None:
            break
        parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
    return [ranks[p] for p in parts]


def _py_encode(ranks, text, eot):
    import regex
    pat = regex.compile(GPT2_SPLIT_PATTERN)
    ids = []
    for k, part in enumerate(text.split("<|endoftext|>")):
        if k:
            ids.append(eot)
        for piece in pat.findall(part):
            ids += _py_merge(ranks, piece.encode())
    return ids


@pytest.fixture(scope="module")
def tok():
    ranks = _table()
    assert len(ranks) > 270  # 256 bytes and a few dozen merges
    return Gpt2Tokenizer(ranks=ranks, endoftext_id=len(ranks) + 7), ranks


TEXTS = ["the quick brown fox", " the  dog's   things!!!\n\nthey're here 1234", "", " ", "a", "\n", "  \t \n x",
         "don't can't I'll we've I'm he'd it's 'tis", "x<|endoftext|>y<|endoftext|>", "hello world 2024-11-25 $3.50",
         "naïve café über 中文 — €5 ½ \U0001F600 ok", "tabs\tand\r\nCRLF  ", "!!!???...", "A" * 300]


@pytest.mark.parametrize("text", TEXTS)
def test_encode_matches_the_published_algorithm_and_round_trips(tok, text):
    t, ranks = tok
    ids = t.encode(text)
    assert ids == _py_encode(ranks, text, t.endoftext_id)
    assert t.decode(ids) == text
    native = t.encode_native(text)
    assert t.decode(native) == text  # whatever the split, the bytes come back
    if all(ord(c) < 128 for c in text):
        assert native == ids  # the library's own splitter is exact on ASCII


@settings(max_examples=150, deadline=None)
@given(st.text(max_size=80))
def test_round_trip_property(text):
    ranks = _table()
    t = Gpt2Tokenizer(ranks=ranks, endoftext_id=len(ranks))
    assert t.decode_bytes(t.encode(text)) == text.encode("utf-8")
    assert t.decode_bytes(t.encode_native(text)) == text.encode("utf-8")
    assert t.encode(text) == _py_encode(ranks, text, t.endoftext_id)


def test_vocabulary_file_in_tiktoken_format(tmp_path, tok):
    t, ranks = tok
    p = tmp_path / "toy.tiktoken"
    p.write_text("".join(f"{base64.b64encode(b).decode()} {r}\n" for b, r in ranks.items()))
    t2 = Gpt2Tokenizer(p, endoftext_id=t.endoftext_id)
    assert t2.vocab_size() == t.vocab_size() == t.endoftext_id + 1
    s = " the quick brown fox's 1234 things<|endoftext|>"
    assert t2.encode(s) == t.encode(s) and t2.encode(s)[-1] == t.endoftext_id


def test_errors(tmp_path, tok):
    t, ranks = tok
    with pytest.raises(TokenizerError):
        Gpt2Tokenizer(tmp_path / "missing.tiktoken")
    bad = tmp_path / "bad.tiktoken"
    bad.write_text("!!!notbase64 3\n")
    with pytest.raises(TokenizerError):
        Gpt2Tokenizer(bad)
    few = dict(list(ranks.items())[:200])  # not every single byte is a token
    with pytest.raises(TokenizerError):
        Gpt2Tokenizer(ranks=few)
    with pytest.raises(TokenizerError):
        t.decode([10 ** 6])  # an id outside the vocabulary
    lone = [ranks[bytes([0xC3])]]  # half of a two-byte sequence: bytes come back, text does not
    assert t.decode_bytes(lone) == b"\xc3"
    with pytest.raises(TokenizerError):
        t.decode(lone)
    with pytest.raises(TokenizerError):
        Gpt2Tokenizer()
