"""Byte-level BPE tokenizer with the reference's behaviour and file format (ai/data/tokenizer.lua), and the
id batches that feed the device-resident model: the step before the token loop.

Same rules as the reference: chunks from ` ?%a+ | ?%d+ | ?[^%s%w]+ | %s+` (C locale, so every byte >= 0x80
is punctuation), merges learned on chunk frequencies with (count, then length-prefixed key) priority and
min_frequency cut-off, vocabulary = special tokens, the 256 bytes, merged strings; `encode` applies the
lowest-rank adjacent merge one occurrence at a time; `decode` drops special tokens and unknown ids; `save` /
`load` use the versioned "bpe\\t2" text format with C-style escapes.  Ids are 1-based, as in the reference;
`to_device_ids` converts to the zero-based int32 the C ABI takes.

Strings may be given as `str` (encoded as UTF-8) or `bytes`; tokens are bytes throughout.

`train()` is deterministic here - distinct chunks are numbered in order of first appearance and the chunks
touched by a merge are visited in ascending order - where the reference walks two Lua hash tables
(tokenizer.lua:222-228, 297-299); on inputs where that order matters the reference's merges depend on the
Lua implementation.
"""
import heapq
import os
import re

import numpy as np

FORMAT_VERSION = 2                                         # tokenizer.lua:8
_WS = rb" \t\n\r\f\v"                                    # %s of the C locale, as a regex class body
_WS_BYTES = b" \t\n\r\f\v"                              # the same six bytes
_CHUNK = re.compile(rb" ?[A-Za-z]+| ?[0-9]+| ?[^" + _WS + rb"A-Za-z0-9]+|[" + _WS + rb"]+|.", re.DOTALL)
_BLOCK = 1024 * 256                                        # tokenizer.lua:195


class TokenizerError(ValueError):
    pass


def _b(s):
    if isinstance(s, str):
        return s.encode("utf-8")
    if isinstance(s, (bytes, bytearray, memoryview)):
        return bytes(s)
    raise TypeError("expected a string, got " + type(s).__name__)


def pretokenize(text):
    """Chunks of `text` in order (tokenizer.lua:10-24)."""
    return _CHUNK.findall(_b(text))


_ESCAPE = {0x5C: b"\\\\", 0x0A: b"\\n", 0x0D: b"\\r", 0x09: b"\\t"}
_ESC_RE = re.compile(rb"[\x00-\x1f\x7f\\]")


def escape(s):
    """Control bytes and the backslash as \\n \\r \\t \\\\ or \\xHH (tokenizer.lua:26-33)."""
    return _ESC_RE.sub(lambda m: _ESCAPE.get(m.group()[0], b"\\x%02X" % m.group()[0]), s)


def unescape(s):
    """Inverse of `escape`; an unknown escape or a bad \\x pair is an error (tokenizer.lua:35-61)."""
    if b"\\" not in s:
        return s
    out, i, n = bytearray(), 0, len(s)
    simple = {0x6E: 0x0A, 0x72: 0x0D, 0x74: 0x09, 0x5C: 0x5C}            # n r t backslash
    while i < n:
        c = s[i]
        if c != 0x5C:
            out.append(c)
            i += 1
            continue
        nx = s[i + 1] if i + 1 < n else None
        if nx in simple:
            out.append(simple[nx])
            i += 2
        elif nx == 0x78:                                                    # x: two characters, both hexadecimal
            try:
                out.append(int(s[i + 2:i + 4].decode("latin-1"), 16))
            except ValueError:
                raise TokenizerError("tokenizer: bad \\x escape in merge file")
            i += 4
        else:
            raise TokenizerError("tokenizer: unknown escape '\\" + (chr(nx) if nx is not None else "") + "' in merge file")
    return bytes(out)


def _key(a, b):
    """Tie-break key of a pair: decimal length of a, \\x01, a, b - compared bytewise (tokenizer.lua:66-73)."""
    return b"%d\x01" % len(a) + a + b


class Tokenizer:
    """Mirror of the reference's tokenizer object: new(config) / train / encode / decode / save / load."""

    def __init__(self, config=None, **kw):
        cfg = dict(config or {}, **kw)
        self.text = cfg.get("text")
        self.text_file = cfg.get("text_file")
        self.vocab_size = cfg.get("vocab_size", 500)
        self.min_frequency = cfg.get("min_frequency", 2)
        sp = cfg.get("special_tokens")
        self.special_tokens = [_b(t) for t in (["<pad>", "<s>", "</s>", "<unk>"] if sp is None else sp)]
        self.log_every = cfg.get("log_every", 50)
        self.verbose = bool(cfg.get("verbose", False))          # the reference prints by default; a library does not
        self.merges = []
        self.trained = False
        self._memo = {}

    new = classmethod(lambda cls, config=None, **kw: cls(config, **kw))

    def target_merges(self):
        """Merges still to learn: vocab_size minus the special tokens and the 256 bytes (tokenizer.lua:168-173)."""
        return max(0, self.vocab_size - (len(self.special_tokens) + 256))

    # ---- vocabulary ---------------------------------------------------------------------------------------
    def _rebuild_vocab(self):
        """tokenizer.lua:116-143: specials, bytes, merged strings; a string that comes up twice keeps its first id;
        the rank of a pair is the first merge that names it."""
        self.vocab, self.inv_vocab, self._rank = {}, [None], {}
        for t in list(self.special_tokens) + [bytes([i]) for i in range(256)] + [a + b for a, b in self.merges]:
            if t not in self.vocab:
                self.vocab[t] = len(self.inv_vocab)
                self.inv_vocab.append(t)
        for i, pair in enumerate(self.merges, start=1):
            self._rank.setdefault(pair, i)
        self.vocab_size = len(self.inv_vocab) - 1
        self.unk_id = self.vocab.get(b"<unk>")
        self._memo = {}
        self._specials = frozenset(self.special_tokens)
        self.trained = True
        return self

    # ---- training -----------------------------------------------------------------------------------------
    def _collect(self):
        """Chunk frequencies of `text`, or of `text_file` read in 256 KB blocks cut at the last whitespace byte
        (tokenizer.lua:184-215; the cut makes a chunk boundary that the whole text would not have)."""
        freqs = {}
        def count(piece):
            for c in _CHUNK.findall(piece):
                freqs[c] = freqs.get(c, 0) + 1
        if self.text is not None:
            count(_b(self.text))
        elif self.text_file is not None:
            try:
                f = open(self.text_file, "rb")
            except OSError:
                raise TokenizerError("tokenizer: cannot open text_file '%s'" % (self.text_file,))
            with f:
                carry = b""
                while True:
                    block = f.read(_BLOCK)
                    if not block:
                        break
                    block = carry + block
                    cut = len(block)
                    while cut > 0 and block[cut - 1] not in _WS_BYTES:
                        cut -= 1
                    if cut == 0:
                        carry = block
                    else:
                        count(block[:cut])
                        carry = block[cut:]
                if carry:
                    count(carry)
        else:
            raise TokenizerError("tokenizer: need config.text or config.text_file")
        return freqs

    def train(self):
        """Learn merges from the configured text (tokenizer.lua:217-345).

        Pair counts are kept incrementally.  The heap holds (count, key) entries; an entry is live only while its count
        equals the pair's current count.  As in the reference, a pair is pushed when a rebuilt chunk re-adds it, not when
        a merge next to it lowers its count, so a pair whose last change was such a decrement is not drawn again until
        some chunk re-adds it."""
        self.merges = []
        freqs = self._collect()
        words = [[bytes([x]) for x in w] for w in freqs]            # first-appearance order
        wfreq = list(freqs.values())
        counts, where = {}, {}

        def bump(pair, delta, widx):
            cur = counts.get(pair, 0) + delta
            if cur <= 0:
                counts.pop(pair, None)
                where.pop(pair, None)
            else:
                counts[pair] = cur
                ws = where.setdefault(pair, set())
                if widx is not None:
                    ws.add(widx)
            return cur

        for i, t in enumerate(words):
            for j in range(len(t) - 1):
                bump((t[j], t[j + 1]), wfreq[i], i)
        heap = [(-c, _key(a, b), a, b) for (a, b), c in counts.items()]
        heapq.heapify(heap)
        want = self.target_merges()
        while len(self.merges) < want:
            top = None
            while heap:
                negc, _, a, b = heapq.heappop(heap)
                if counts.get((a, b)) == -negc:
                    top = (-negc, a, b)
                    break
            if top is None or top[0] < self.min_frequency:
                break
            _, a, b = top
            merged = a + b
            self.merges.append((a, b))
            for widx in sorted(where.get((a, b), ())):
                t, fq = words[widx], wfreq[widx]
                nt, j, n = [], 0, len(t)
                while j < n:
                    if j < n - 1 and t[j] == a and t[j + 1] == b:
                        nt.append(merged)
                        j += 2
                    else:
                        nt.append(t[j])
                        j += 1
                if len(nt) == n:                                   # the pair is no longer in this chunk
                    continue
                for j in range(n - 1):
                    bump((t[j], t[j + 1]), -fq, None)
                words[widx] = nt
                for j in range(len(nt) - 1):
                    p = (nt[j], nt[j + 1])
                    heapq.heappush(heap, (-bump(p, fq, widx), _key(*p), p[0], p[1]))
            counts.pop((a, b), None)
            where.pop((a, b), None)
            if self.verbose and len(self.merges) % self.log_every == 0:
                print("Merge #%d: %r + %r (count=%d)" % (len(self.merges), a, b, top[0]))
        self._rebuild_vocab()
        if self.verbose:
            print("Vocabulary: %d tokens from %d merges" % (self.vocab_size, len(self.merges)))
        return self

    # ---- encode / decode ----------------------------------------------------------------------------------
    def _bpe(self, chunk):
        """Tokens of one chunk: merge the adjacent pair of lowest rank, leftmost on ties, one occurrence at a time
        (tokenizer.lua:347-373).  Memoised per chunk."""
        hit = self._memo.get(chunk)
        if hit is not None:
            return hit
        toks = [bytes([x]) for x in chunk]
        rank = self._rank
        while len(toks) > 1:
            best, at = None, -1
            for i in range(len(toks) - 1):
                r = rank.get((toks[i], toks[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            toks[at:at + 2] = [toks[at] + toks[at + 1]]
        self._memo[chunk] = toks
        return toks

    def encode(self, text):
        """1-based ids of `text` (tokenizer.lua:375-398)."""
        if not self.trained:
            raise TokenizerError("tokenizer:encode: tokenizer has no vocabulary yet, call :train() or :load() first")
        if not isinstance(text, (str, bytes, bytearray, memoryview)):
            raise TokenizerError("tokenizer:encode: expected a string, got " + type(text).__name__)
        vocab, unk, out = self.vocab, self.unk_id, []
        for chunk in _CHUNK.findall(_b(text)):
            for t in self._bpe(chunk):
                i = vocab.get(t, unk)
                if i is None:
                    raise TokenizerError("tokenizer:encode: token %r is not in the vocabulary and there is no <unk>" % (t,))
                out.append(i)
        return out

    def decode(self, tokens):
        """Bytes of the 1-based ids; special tokens and ids outside the vocabulary are dropped (tokenizer.lua:400-415)."""
        if not self.trained:
            raise TokenizerError("tokenizer:decode: tokenizer has no vocabulary yet, call :train() or :load() first")
        inv, sp, n = self.inv_vocab, self._specials, len(self.inv_vocab)
        return b"".join(inv[int(i)] for i in tokens if 1 <= int(i) < n and inv[int(i)] not in sp)

    def decode_text(self, tokens, errors="replace"):
        return self.decode(tokens).decode("utf-8", errors)

    # ---- file format --------------------------------------------------------------------------------------
    def dumps(self):
        """The bytes `save` writes: "bpe\\t2", the special tokens, the merges, escaped (tokenizer.lua:417-434)."""
        lines = [b"bpe\t%d" % FORMAT_VERSION, b"specials\t%d" % len(self.special_tokens)]
        lines += [escape(t) for t in self.special_tokens]
        lines.append(b"merges\t%d" % len(self.merges))
        lines += [escape(a) + b"\t" + escape(b) for a, b in self.merges]
        return b"\n".join(lines) + b"\n"

    def save(self, path):
        try:
            with open(path, "wb") as f:
                f.write(self.dumps())
        except OSError as e:
            raise TokenizerError("tokenizer:save: cannot write '%s': %s" % (path, e))
        return self

    def loads(self, data, path="<bytes>"):
        """Parse the saved format with the reference's checks and messages (tokenizer.lua:436-492)."""
        lines = data.split(b"\n")
        if lines and lines[-1] == b"":
            lines.pop()                                           # io.lines yields no empty last line
        it = iter(lines)
        m = re.fullmatch(rb"([A-Za-z]+)\t([0-9]+)", next(it, b""))
        if not m or m.group(1) != b"bpe":
            raise TokenizerError("tokenizer:load: '%s' is not a versioned bpe file (re-train and :save() to upgrade the old "
                                 "lossy format)" % path)
        if int(m.group(2)) > FORMAT_VERSION:
            raise TokenizerError("tokenizer:load: file format v%d is newer than supported v%d" % (int(m.group(2)), FORMAT_VERSION))
        m = re.fullmatch(rb"specials\t([0-9]+)", next(it, b""))
        if not m:
            raise TokenizerError("tokenizer:load: missing specials header")
        specials = [unescape(next(it, b"")) for _ in range(int(m.group(1)))]
        m = re.fullmatch(rb"merges\t([0-9]+)", next(it, b""))
        if not m:
            raise TokenizerError("tokenizer:load: missing merges header")
        merges, nmerge = [], int(m.group(1))
        for i in range(nmerge):
            line = next(it, None)
            if line is None:
                raise TokenizerError("tokenizer:load: file ends after %d of %d merges" % (i, nmerge))
            a, tab, b = line.partition(b"\t")
            if not tab:
                raise TokenizerError("tokenizer:load: malformed merge on line %d" % (3 + len(specials) + i + 1))
            merges.append((unescape(a), unescape(b)))
        self.special_tokens, self.merges = specials, merges
        return self._rebuild_vocab()

    def load(self, path):
        try:
            with open(path, "rb") as f:
                data = f.read()
        except OSError as e:
            raise TokenizerError("tokenizer:load: cannot open '%s': %s" % (path, e))
        return self.loads(data, os.fspath(path))


# ---- byte-level ids (no tokenizer) ------------------------------------------------------------------------
def byte_encode(text):
    """Ids 1..256 of the bytes of `text`: the reference's fallback when no tokenizer is set (lmtrain.lua:190-197)."""
    if not isinstance(text, (str, bytes, bytearray, memoryview)):
        raise TokenizerError("LMTrain.encode: expected a string, got " + type(text).__name__)
    return (np.frombuffer(_b(text), dtype=np.uint8).astype(np.int32) + 1).tolist()


def byte_decode(tokens):
    """Inverse of `byte_encode`; an id outside 1..256 is an error, as in the reference (lmtrain.lua:199-212)."""
    out = bytearray()
    for i, t in enumerate(tokens, start=1):
        if not isinstance(t, (int, np.integer)) or t < 1 or t > 256:
            raise TokenizerError("LMTrain.decode: token %d = %s cannot be a byte (need 1..256); this model's vocab is larger "
                                 "than a byte alphabet" % (i, t))
        out.append(int(t) - 1)
    return bytes(out)


# ---- ids -> the blocks the device step takes --------------------------------------------------------------
def to_device_ids(ids, zero_indexed=True):
    """int32 array of the ids, shifted to the zero-based ids of the C ABI unless zero_indexed is False."""
    a = np.asarray(ids, dtype=np.int64)
    return np.ascontiguousarray(a - 1 if zero_indexed else a, dtype=np.int32)


def build_windows(sequences, max_seq, stride=None):
    """Training windows of every id sequence: inputs seq[start : stop], targets shifted by one, at most max_seq long,
    starts `stride` apart (default max_seq), the last window of a sequence ending at its last id (lmtrain.lua:535-558).
    Returns (inp, tgt, n) triples of 1-based int32 arrays."""
    stride = stride or max_seq
    out = []
    for seq in sequences:
        s = np.asarray(seq, dtype=np.int32)
        n_seq, start = len(s), 0
        while start < n_seq - 1:
            stop = min(start + max_seq, n_seq - 1)
            out.append((s[start:stop], s[start + 1:stop + 1], stop - start))
            if stop >= n_seq - 1:
                break
            start += stride
    return out


class IdBatches:
    """Blocks of `batch` windows in the layout of the device training step: zero-based int32 ids [batch, seq_len]
    (pad 0) and targets (pad -1), written into one reusable host buffer - page-locked when a CUDA device is
    present, so that the copy to the device is a DMA from the buffer itself - plus the number of valid targets.
    Ids outside 1..vocab are an error, with the reference's message (gpu_transformer.lua:_pack)."""

    def __init__(self, windows, batch, seq_len, vocab, pinned=None):
        self.windows, self.B, self.T, self.V = windows, int(batch), int(seq_len), int(vocab)
        self.pinned, self._host = False, None
        buf = None
        if pinned is not False:
            # page-locked memory from the backend itself (the reference's luaTL_host_alloc_pinned,
            # cuda/luaTL_core.cu:1801), once luaTL_init has bound a device
            try:
                import ctypes as C
                from . import _lib
                _lib.ensure_init()
                nbytes = 2 * self.B * self.T * 4
                ptr = _lib.load().luaTL_host_alloc_pinned(nbytes)
                if not ptr:
                    raise TokenizerError("IdBatches: " + _lib.last_error())
                self._host = ptr
                flat = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_int32)), shape=(2 * self.B * self.T,))
                buf, self.pinned = flat.reshape(2, self.B, self.T), True
            except Exception:
                if pinned:
                    raise TokenizerError("IdBatches: page-locked memory needs a CUDA device")
        if buf is None:
            buf = np.empty((2, self.B, self.T), dtype=np.int32)
        self.ids, self.tgt = buf[0], buf[1]

    def __len__(self):
        return (len(self.windows) + self.B - 1) // self.B

    def close(self):
        """Give the page-locked buffer back (views of it must not be used afterwards)."""
        if self._host:
            from . import _lib
            self.ids = self.tgt = None
            _lib.load().luaTL_host_free_pinned(self._host)
            self._host, self.pinned = None, False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def fill(self, first):
        """Pack windows[first : first + batch]; returns (ids, tgt, valid) - views of the reusable buffer."""
        self.ids.fill(0)
        self.tgt.fill(-1)
        valid = 0
        for b, w in enumerate(self.windows[first:first + self.B]):
            n = min(int(w[2]) if len(w) > 2 and w[2] else len(w[0]), self.T)
            inp, tg = np.asarray(w[0][:n], dtype=np.int64), np.asarray(w[1][:n], dtype=np.int64)
            bad = np.flatnonzero((inp < 1) | (inp > self.V) | (tg < 1) | (tg > self.V))
            if bad.size:
                t = int(bad[0])
                raise ValueError("gpu_transformer: token out of range at window %d, pos %d (input %d, target %d, vocab %d)"
                                 % (first + b + 1, t + 1, inp[t], tg[t], self.V))
            self.ids[b, :n], self.tgt[b, :n] = inp - 1, tg - 1
            valid += n
        return self.ids, self.tgt, valid

    def __iter__(self):
        for first in range(0, len(self.windows), self.B):
            yield self.fill(first)
