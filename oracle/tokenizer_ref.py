"""TEST INFRASTRUCTURE - a literal CPU restatement of the reference's byte-level BPE tokenizer
(ai/data/tokenizer.lua), used only by tests/ to check lanternl_b200/tokenizer.py.

Everything works on bytes, as Lua strings do; ids are 1-based, as the reference's are.
Each function names the reference lines it follows.

Parity status: pinned by the reference's own test (tests/core_test.lua:63-70: train on "hello world"
with vocab_size 100 -> no merges, ids are specials + bytes) and by vectors derived by hand from the
source text; no Lua runtime exists in the build environment to run tokenizer.lua itself, so beyond
those the restatement is "parity unpinned".

One part of the reference is not a function of its input: train() numbers the distinct chunks in
the order of pairs(freqs) and visits the chunks touched by a merge in the order of pairs(affected)
(tokenizer.lua:222-228, 297-299), both hash orders of the Lua implementation.  The order decides
whether the last operation on a neighbouring pair is a pushed increment or an unpushed decrement
(tokenizer.lua:311-329), i.e. whether that pair can still be drawn from the heap.  The restatement
fixes the order - chunks numbered by first appearance, touched chunks ascending - and says so here.
"""

FORMAT_VERSION = 2                      # tokenizer.lua:8

_SPACE = frozenset(b" \t\n\v\f\r")      # %s in the C locale
_ALPHA = frozenset(range(65, 91)) | frozenset(range(97, 123))
_DIGIT = frozenset(range(48, 58))


def _run(s, i, cls, negate=False):
    """End (exclusive) of the longest run of bytes in (or outside) cls starting at i."""
    n = len(s)
    j = i
    while j < n and ((s[j] in cls) != negate):
        j += 1
    return j


def pretokenize(s):
    """tokenizer.lua:10-24 - ' ?%a+', else ' ?%d+', else ' ?[^%s%w]+', else '%s+', else one byte."""
    out = []
    i, n = 0, len(s)
    alnum_space = _SPACE | _ALPHA | _DIGIT
    while i < n:
        en = None
        for cls, neg in ((_ALPHA, False), (_DIGIT, False), (alnum_space, True)):
            # ' ?X+': try with the optional space taken, then (backtracking) without it
            if s[i] == 0x20:
                e = _run(s, i + 1, cls, neg)
                if e > i + 1:
                    en = e
                    break
            e = _run(s, i, cls, neg)
            if e > i:
                en = e
                break
        if en is None:
            e = _run(s, i, _SPACE)
            en = e if e > i else i + 1
        out.append(bytes(s[i:en]))
        i = en
    return out


_ESC = {0x5C: b"\\\\", 0x0A: b"\\n", 0x0D: b"\\r", 0x09: b"\\t"}


def escape(s):
    """tokenizer.lua:26-33 - control bytes (%c: 0..31 and 127) and the backslash."""
    out = bytearray()
    for c in s:
        if c in _ESC:
            out += _ESC[c]
        elif c < 32 or c == 127:
            out += b"\\x%02X" % c
        else:
            out.append(c)
    return bytes(out)


def unescape(s):
    """tokenizer.lua:35-61."""
    out = bytearray()
    i, n = 0, len(s)
    while i < n:
        c = s[i]
        if c == 0x5C:
            nx = s[i + 1:i + 2]
            if nx == b"n":
                out.append(0x0A); i += 2
            elif nx == b"r":
                out.append(0x0D); i += 2
            elif nx == b"t":
                out.append(0x09); i += 2
            elif nx == b"\\":
                out.append(0x5C); i += 2
            elif nx == b"x":
                try:
                    out.append(int(s[i + 2:i + 4].decode("latin-1"), 16))
                except ValueError:
                    raise ValueError("tokenizer: bad \\x escape in merge file")
                i += 4
            else:
                raise ValueError("tokenizer: unknown escape '\\" + nx.decode("latin-1") + "' in merge file")
        else:
            out.append(c)
            i += 1
    return bytes(out)


def heap_key(a, b):
    """tokenizer.lua:66-68 - '%d\\1%s%s' of (#a, a, b); compared bytewise (C locale)."""
    return str(len(a)).encode() + b"\x01" + a + b


class Heap:
    """tokenizer.lua:63-114 - binary heap on (count descending, key ascending), 1-based like the source."""

    def __init__(self):
        self.e = [None]

    @staticmethod
    def better(x, y):
        if x[0] != y[0]:
            return x[0] > y[0]
        return x[3] < y[3]

    def push(self, c, a, b):
        self.e.append((c, a, b, heap_key(a, b)))
        n = len(self.e) - 1
        while n > 1:
            parent = n // 2
            if self.better(self.e[n], self.e[parent]):
                self.e[n], self.e[parent] = self.e[parent], self.e[n]
                n = parent
            else:
                break

    def pop(self):
        n = len(self.e) - 1
        if n == 0:
            return None
        top = self.e[1]
        self.e[1] = self.e[n]
        self.e.pop()
        n -= 1
        i = 1
        while True:
            l, r, best = 2 * i, 2 * i + 1, i
            if l <= n and self.better(self.e[l], self.e[best]):
                best = l
            if r <= n and self.better(self.e[r], self.e[best]):
                best = r
            if best == i:
                break
            self.e[i], self.e[best] = self.e[best], self.e[i]
            i = best
        return top


class Tokenizer:
    DEFAULT_SPECIALS = (b"<pad>", b"<s>", b"</s>", b"<unk>")

    def __init__(self, text=None, vocab_size=500, min_frequency=2, special_tokens=None):
        """tokenizer.lua:145-162."""
        self.text = text
        self.vocab_size = vocab_size
        self.min_frequency = min_frequency
        self.special_tokens = list(self.DEFAULT_SPECIALS if special_tokens is None else special_tokens)
        self.merges = []
        self.trained = False

    def target_merges(self):
        """tokenizer.lua:168-173."""
        return max(0, self.vocab_size - (len(self.special_tokens) + 256))

    def rebuild_vocab(self):
        """tokenizer.lua:116-143 - specials, the 256 bytes, then the merged strings; a string seen twice keeps its first id."""
        self.vocab, self.inv_vocab, self.ranks = {}, [None], {}
        def add(t):
            if t not in self.vocab:
                self.inv_vocab.append(t)
                self.vocab[t] = len(self.inv_vocab) - 1
        for t in self.special_tokens:
            add(t)
        for i in range(256):
            add(bytes([i]))
        for i, (a, b) in enumerate(self.merges, start=1):
            add(a + b)
            self.ranks.setdefault(a, {}).setdefault(b, i)
        self.vocab_size = len(self.inv_vocab) - 1
        self.unk_id = self.vocab.get(b"<unk>")
        self.trained = True
        return self

    def train(self):
        """tokenizer.lua:217-345, chunks numbered by first appearance and touched chunks visited ascending."""
        self.merges = []
        freqs = {}
        for c in pretokenize(self.text):
            freqs[c] = freqs.get(c, 0) + 1
        words = [None] + [[bytes([x]) for x in w] for w in freqs]
        wfreq = [None] + list(freqs.values())
        counts, where = {}, {}

        def bump(a, b, delta, widx):
            ca = counts.setdefault(a, {})
            cur = ca.get(b, 0) + delta
            if cur <= 0:
                ca.pop(b, None)
                if a in where:
                    where[a].pop(b, None)
            else:
                ca[b] = cur
                wb = where.setdefault(a, {}).setdefault(b, set())
                if widx is not None:
                    wb.add(widx)
            return cur

        for i in range(1, len(words)):
            t = words[i]
            for j in range(len(t) - 1):
                bump(t[j], t[j + 1], wfreq[i], i)
        heap = Heap()
        for a, row in counts.items():
            for b, c in row.items():
                heap.push(c, a, b)
        want = self.target_merges()
        while len(self.merges) < want:
            while True:
                top = heap.pop()
                if top is None:
                    break
                cur = counts.get(top[1], {}).get(top[2])
                if cur is not None and cur == top[0]:
                    break
            if top is None or top[0] < self.min_frequency:
                break
            a, b = top[1], top[2]
            merged = a + b
            self.merges.append((a, b))
            for widx in sorted(where.get(a, {}).get(b, ())):
                t, fq = words[widx], wfreq[widx]
                if not any(t[j] == a and t[j + 1] == b for j in range(len(t) - 1)):
                    continue
                for j in range(len(t) - 1):
                    bump(t[j], t[j + 1], -fq, None)
                nt, j = [], 0
                while j < len(t):
                    if j < len(t) - 1 and t[j] == a and t[j + 1] == b:
                        nt.append(merged); j += 2
                    else:
                        nt.append(t[j]); j += 1
                words[widx] = nt
                for j in range(len(nt) - 1):
                    heap.push(bump(nt[j], nt[j + 1], fq, widx), nt[j], nt[j + 1])
            counts.get(a, {}).pop(b, None)
            where.get(a, {}).pop(b, None)
        return self.rebuild_vocab()

    def bpe(self, chunk):
        """tokenizer.lua:347-373 - merge the adjacent pair of lowest rank (leftmost on ties), one occurrence at a time."""
        toks = [bytes([x]) for x in chunk]
        while len(toks) > 1:
            best_rank, best_i = None, None
            for i in range(len(toks) - 1):
                r = self.ranks.get(toks[i], {}).get(toks[i + 1])
                if r is not None and (best_rank is None or r < best_rank):
                    best_rank, best_i = r, i
            if best_i is None:
                break
            toks[best_i:best_i + 2] = [toks[best_i] + toks[best_i + 1]]
        return toks

    def encode(self, text):
        """tokenizer.lua:375-398."""
        if not self.trained:
            raise RuntimeError("tokenizer:encode: tokenizer has no vocabulary yet, call :train() or :load() first")
        out = []
        for chunk in pretokenize(text):
            for t in self.bpe(chunk):
                i = self.vocab.get(t, self.unk_id)
                if i is None:
                    raise RuntimeError("tokenizer:encode: token is not in the vocabulary and there is no <unk>")
                out.append(i)
        return out

    def decode(self, tokens):
        """tokenizer.lua:400-415 - ids outside the vocabulary and special tokens are dropped."""
        if not self.trained:
            raise RuntimeError("tokenizer:decode: tokenizer has no vocabulary yet, call :train() or :load() first")
        sp = set(self.special_tokens)
        out = []
        for i in tokens:
            t = self.inv_vocab[i] if isinstance(i, int) and 1 <= i < len(self.inv_vocab) else None
            if t is not None and t not in sp:
                out.append(t)
        return b"".join(out)

    def dumps(self):
        """tokenizer.lua:417-434 - the bytes save() writes."""
        lines = [b"bpe\t%d" % FORMAT_VERSION, b"specials\t%d" % len(self.special_tokens)]
        lines += [escape(t) for t in self.special_tokens]
        lines.append(b"merges\t%d" % len(self.merges))
        lines += [escape(a) + b"\t" + escape(b) for a, b in self.merges]
        return b"\n".join(lines) + b"\n"
