"""The BPE tokenizer and the id batches in front of the token loop (CPU only): the reference's own test case,
vectors derived by hand from ai/data/tokenizer.lua, the saved file byte for byte, the module against the
literal restatement in oracle/ on seeded corpora, error messages, windows and batch packing."""
import os

import numpy as np
import pytest

from lanternl_b200 import tokenizer as T
from oracle import tokenizer_ref as R


def corpus(seed, nwords=400, alphabet=b"abcdeio nt", extra=(b"12", b"!?", b"\n", b"\xc3\xa9", b"  ")):
    rng = np.random.default_rng(seed)
    parts = []
    for _ in range(nwords):
        if rng.random() < 0.1:
            parts.append(extra[rng.integers(len(extra))])
        else:
            n = int(rng.integers(1, 7))
            parts.append(bytes(alphabet[i] for i in rng.integers(0, len(alphabet), n)))
        parts.append(b" ")
    return b"".join(parts)


def test_reference_round_trip_case():
    """tests/core_test.lua:63-70: "hello world" with vocab_size 100 leaves no room for merges; ids are bytes + 5."""
    tok = T.Tokenizer.new(dict(text="hello world", vocab_size=100)).train()
    assert tok.target_merges() == 0 and tok.merges == [] and tok.vocab_size == 260
    ids = tok.encode("hello")
    assert ids == [109, 106, 113, 113, 116]
    assert tok.decode(ids) == b"hello" and tok.decode_text(ids) == "hello"
    assert [tok.vocab[t] for t in (b"<pad>", b"<s>", b"</s>", b"<unk>")] == [1, 2, 3, 4] and tok.unk_id == 4


def test_reference_example_script_case():
    """examples/train_tokenizer.lua: the same vocab_size 100 on a longer text - still no merges; the saved file is the header alone."""
    tok = T.Tokenizer.new(dict(text="hello world, this is a test of the lanternl tokenizer. it learns words and subwords.",
                               vocab_size=100, verbose=False)).train()
    ids = tok.encode("hello world")
    assert ids == [b + 5 for b in b"hello world"] and tok.decode(ids) == b"hello world"
    assert tok.dumps() == b"bpe\t2\nspecials\t4\n<pad>\n<s>\n</s>\n<unk>\nmerges\t0\n"


@pytest.mark.parametrize("text,chunks", [
    (b"hello world", [b"hello", b" world"]),
    (b"a  b", [b"a", b"  ", b"b"]),                           # two blanks: the run of blanks wins over ' ?%a+'
    (b"x1 23!! ok", [b"x", b"1", b" 23", b"!!", b" ok"]),
    (b" \n x", [b" \n ", b"x"]),
    (b"caf\xc3\xa9 _a", [b"caf", b"\xc3\xa9", b" _", b"a"]),     # bytes >= 0x80 and '_' are punctuation in the C locale
    (b"a\x00b", [b"a", b"\x00", b"b"]),
    (b"", []),
])
def test_pretokenize_rules(text, chunks):
    assert T.pretokenize(text) == chunks == R.pretokenize(text)


def test_escape_round_trip_and_errors():
    raw = bytes(range(256))
    assert T.unescape(T.escape(raw)) == raw
    assert T.escape(b"a\tb\\c\n\r\x01\x7f\xff") == b"a\\tb\\\\c\\n\\r\\x01\\x7F\xff" == R.escape(b"a\tb\\c\n\r\x01\x7f\xff")
    with pytest.raises(T.TokenizerError, match="unknown escape"):
        T.unescape(b"a\\q")
    with pytest.raises(T.TokenizerError, match="unknown escape"):
        T.unescape(b"trailing\\")
    with pytest.raises(T.TokenizerError, match=r"bad \\x escape"):
        T.unescape(b"\\xZ1")


def test_hand_derived_merges_ids_and_file():
    """"ab ab ab abc": chunks ab x1, ' ab' x2, ' abc' x1 -> (a,b) 4 times, then (' ', ab) 3 times."""
    tok = T.Tokenizer(text="ab ab ab abc", vocab_size=262).train()
    assert tok.merges == [(b"a", b"b"), (b" ", b"ab")]
    assert tok.vocab[b"ab"] == 261 and tok.vocab[b" ab"] == 262 and tok.vocab_size == 262
    assert tok.encode("ab ab abc") == [261, 262, 262, 104]
    assert tok.dumps() == b"bpe\t2\nspecials\t4\n<pad>\n<s>\n</s>\n<unk>\nmerges\t2\na\tb\n \tab\n"


def test_tie_break_and_min_frequency():
    # equal counts: the smaller key "<len a>\1<a><b>" wins, bytewise: ' ' < 'a' < 'c'
    tok = T.Tokenizer(text="ab cd ab cd", vocab_size=261).train()
    assert tok.merges == [(b" ", b"c")]
    # a shorter left part beats a longer one whatever the bytes: "1\1..." < "2\1..."
    tok = T.Tokenizer(text="zzy zzy", vocab_size=262, min_frequency=1).train()
    assert tok.merges[0] == (b"z", b"y") or tok.merges[0] == (b"z", b"z")
    assert T._key(b"z", b"z") > T._key(b"z", b"y") and T._key(b"zz", b"a") > T._key(b"z", b"zz")
    # nothing reaches min_frequency: no merges although there is room
    tok = T.Tokenizer(text="abc", vocab_size=300, min_frequency=2).train()
    assert tok.merges == []


@pytest.mark.parametrize("seed,vocab,minf", [(0, 300, 2), (1, 340, 2), (2, 280, 1), (3, 400, 3), (4, 520, 2)])
def test_module_against_the_literal_restatement(seed, vocab, minf):
    text = corpus(seed)
    a = T.Tokenizer(text=text, vocab_size=vocab, min_frequency=minf).train()
    b = R.Tokenizer(text=text, vocab_size=vocab, min_frequency=minf).train()
    assert a.merges == b.merges and len(a.merges) > 10
    assert a.vocab == b.vocab and a.dumps() == b.dumps()
    probe = corpus(seed + 100, 120)
    ids = a.encode(probe)
    assert ids == b.encode(probe)
    assert a.decode(ids) == probe == b.decode(ids)
    assert len(ids) < len(probe)                                      # the merges are used


def test_save_load_and_special_tokens(tmp_path):
    tok = T.Tokenizer(text=corpus(7), vocab_size=300, special_tokens=["<pad>", "<unk>", "tab\there", "a"]).train()
    assert tok.vocab[b"a"] == 4 and tok.vocab_size == 300 - 1            # the byte 'a' is already a special token
    p = tmp_path / "tok.bpe"
    tok.save(p)
    back = T.Tokenizer().load(p)
    assert back.special_tokens == tok.special_tokens and back.merges == tok.merges and back.vocab == tok.vocab
    ids = tok.encode("a bad tin")
    assert back.encode("a bad tin") == ids
    # decode drops special tokens (here the byte 'a' is one) and ids outside the vocabulary
    assert ids[0] == 4 and tok.decode([1, 2] + ids + [0, 10 ** 6]) == tok.decode(ids) == b" bad tin"


@pytest.mark.parametrize("data,msg", [
    (b"merges\t0\n", "not a versioned bpe file"),
    (b"bpe\t3\nspecials\t0\nmerges\t0\n", "file format v3 is newer than supported v2"),
    (b"bpe\t2\nmerges\t0\n", "missing specials header"),
    (b"bpe\t2\nspecials\t1\n<unk>\n", "missing merges header"),
    (b"bpe\t2\nspecials\t0\nmerges\t2\na\tb\n", "file ends after 1 of 2 merges"),
    (b"bpe\t2\nspecials\t0\nmerges\t1\nab\n", "malformed merge on line 4"),
])
def test_load_errors(data, msg):
    with pytest.raises(T.TokenizerError, match=msg):
        T.Tokenizer().loads(data, "f")


def test_untrained_and_missing_text():
    with pytest.raises(T.TokenizerError, match="no vocabulary yet"):
        T.Tokenizer().encode("x")
    with pytest.raises(T.TokenizerError, match="no vocabulary yet"):
        T.Tokenizer().decode([1])
    with pytest.raises(T.TokenizerError, match="need config.text or config.text_file"):
        T.Tokenizer().train()
    with pytest.raises(T.TokenizerError, match="cannot open text_file"):
        T.Tokenizer(text_file="/nonexistent/corpus.txt").train()


def test_text_file_blocks_cut_at_whitespace(tmp_path, monkeypatch):
    text = corpus(9, 300)
    p = tmp_path / "c.txt"
    p.write_bytes(text)
    whole = T.Tokenizer(text=text, vocab_size=300).train()
    assert T.Tokenizer(text_file=str(p), vocab_size=300).train().merges == whole.merges   # one block: same as the text
    monkeypatch.setattr(T, "_BLOCK", 64)                                 # many blocks: chunks never span a cut
    tok = T.Tokenizer(text_file=str(p), vocab_size=300)
    freqs = tok._collect()
    want, carry, pos = {}, b"", 0
    while pos < len(text):
        block = carry + text[pos:pos + 64]
        pos += 64
        cut = max((i + 1 for i, c in enumerate(block) if c in b" \t\n\r\f\v"), default=0)
        if cut == 0:
            carry = block
            continue
        for c in R.pretokenize(block[:cut]):
            want[c] = want.get(c, 0) + 1
        carry = block[cut:]
    for c in R.pretokenize(carry):
        want[c] = want.get(c, 0) + 1
    assert freqs == want and sum(len(k) * v for k, v in freqs.items()) == len(text)


def test_byte_level_ids():
    assert T.byte_encode("Az") == [66, 123] and T.byte_decode([66, 123]) == b"Az"
    assert T.byte_decode(T.byte_encode(bytes(range(256)))) == bytes(range(256))
    with pytest.raises(T.TokenizerError, match="token 2 = 257 cannot be a byte"):
        T.byte_decode([1, 257])
    assert T.to_device_ids([1, 5, 256]).tolist() == [0, 4, 255] and T.to_device_ids([1, 5], zero_indexed=False).dtype == np.int32


def lua_windows(sequences, max_seq, stride=None):
    """ai/optim/lmtrain.lua:535-558, 1-based as written."""
    stride = stride or max_seq
    out = []
    for seq in sequences:
        ln, start = len(seq), 1
        while start < ln:
            stop = min(start + max_seq, ln)
            inp = [seq[i - 1] for i in range(start, stop)]
            tgt = [seq[i] for i in range(start, stop)]
            if inp:
                out.append((inp, tgt, len(inp)))
            if stop >= ln:
                break
            start += stride
    return out


@pytest.mark.parametrize("lens,max_seq,stride", [([7, 2, 1, 0], 3, None), ([8], 3, None), ([20, 5], 4, 2), ([9], 16, None), ([10], 3, 5)])
def test_windows_follow_the_reference(lens, max_seq, stride):
    rng = np.random.default_rng(3)
    seqs = [rng.integers(1, 50, n).tolist() for n in lens]
    got = T.build_windows(seqs, max_seq, stride)
    want = lua_windows(seqs, max_seq, stride)
    assert [(a.tolist(), b.tolist(), n) for a, b, n in got] == want


def test_id_batches_layout_and_range_check():
    w = T.build_windows([[1, 2, 3, 4, 5, 6, 7], [9, 8]], 3)
    ib = T.IdBatches(w, batch=2, seq_len=3, vocab=10, pinned=False)
    blocks = [(i.copy(), t.copy(), v) for i, t, v in ib]
    assert len(ib) == 2 and not ib.pinned
    assert blocks[0][0].tolist() == [[0, 1, 2], [3, 4, 5]] and blocks[0][1].tolist() == [[1, 2, 3], [4, 5, 6]] and blocks[0][2] == 6
    assert blocks[1][0].tolist() == [[8, 0, 0], [0, 0, 0]] and blocks[1][1].tolist() == [[7, -1, -1], [-1, -1, -1]] and blocks[1][2] == 1
    assert blocks[0][0].dtype == np.int32 and blocks[0][0].flags["C_CONTIGUOUS"]
    with pytest.raises(ValueError, match=r"token out of range at window 3, pos 1 \(input 9, target 8, vocab 8\)"):
        list(T.IdBatches(w, batch=2, seq_len=3, vocab=8, pinned=False))
    if not os.path.exists("/dev/nvidia0"):
        with pytest.raises(T.TokenizerError, match="needs a CUDA device"):
            T.IdBatches(w, 2, 3, 10, pinned=True)


@pytest.mark.gpu
def test_text_to_device_steps_through_page_locked_batches():
    """Text -> BPE ids -> windows -> page-locked [B, T] blocks -> the device training step."""
    from lanternl_b200 import gpu_transformer as GT
    text = corpus(11, 1500)
    tok = T.Tokenizer(text=text, vocab_size=320).train()
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    w = T.build_windows([ids], 32)
    m = GT.new(dict(vocab=tok.vocab_size, dim=32, layers=1, heads=2, ffn=64, max_seq=32, batch_size=8, optimizer="sgd"))
    ib = T.IdBatches(w, batch=8, seq_len=32, vocab=tok.vocab_size)
    assert ib.pinned and len(ib) >= 4
    losses = []
    for epoch in range(3):
        for blk_ids, blk_tgt, valid in ib:
            loss, correct, n, gnorm, finite = m.train_step_ids(blk_ids, blk_tgt, 0.5, m.steps + 1)
            assert finite and n == valid
            losses.append(loss)
    assert losses[-1] < losses[0]
    # the packed blocks are what the window path packs itself
    a, b, _ = m._pack(w[:8], 8)
    i0, t0, _ = ib.fill(0)
    assert np.array_equal(a, i0) and np.array_equal(b, t0)
    ib.close()
    assert not ib.pinned
